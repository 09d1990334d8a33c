// Decode attention: host side (validation, work decomposition, launch), the generic kernels (any
// field width, reference layout, G up to 16) and the partial-merge kernel.
#include <algorithm>
#include <atomic>
#include <mutex>

#include "attn_kernel.cuh"

namespace hqmq {
namespace attn {

const void* fast_kernel(int n_chunks, int ib, int rb, bool outl);
size_t fast_warp_bytes(int n_chunks, int ib, int rb, bool outl);
bool ring_kernel(int n_chunks, int ib, int rb, bool outl, int scale_dtype, RingKernelInfo& k);
size_t ring_smem_total(int table_rows, int repk_log2, int repv_log2, int d, bool outl, int stages, int merge_slots,
                       size_t stage_bytes, int warps);
constexpr int kRingMinKeys = 1024;       // shorter key ranges keep the per-warp staging rings
// ... and so do small problems: below about four stages per SM the ring kernel's set-up (it replicates the tables
// up to sixteen times) outweighs its faster tile loop (B1, 8 KV heads, 4096 keys: 42 against 26 us per step)
constexpr int64_t kRingMinTiles = 148 * 4 * 15;
constexpr size_t kSmemLimit = 226 * 1024;
constexpr int kFastStages = 2;   // must equal kStages of the staged kernels
constexpr int kFastQPad = 8;     // must equal kQPad of the staged kernels

template <int N, bool OUTL, bool WIDE>
__global__ void __launch_bounds__(kSlowWarps * 32) attn_slow_kernel(const AttnParams p) {
  attn_decode_body<N, SlowLoader<N>, kSlowWarps, OUTL, WIDE>(p);
}

template <int N>
static const void* slow_pick(bool outl, bool wide) {
  if (outl) return wide ? (const void*)&attn_slow_kernel<N, true, true> : (const void*)&attn_slow_kernel<N, true, false>;
  return wide ? (const void*)&attn_slow_kernel<N, false, true> : (const void*)&attn_slow_kernel<N, false, false>;
}
static const void* slow_kernel(int n, bool outl, bool wide) {
  switch (n) {
    case 4: return slow_pick<4>(outl, wide);
    case 8: return slow_pick<8>(outl, wide);
    case 12: return slow_pick<12>(outl, wide);
    case 16: return slow_pick<16>(outl, wide);
    case 32: return slow_pick<32>(outl, wide);
    default: return nullptr;
  }
}

// Merge partials: parts [rows][n_parts][d+2] -> normalised output rows, or one merged partial per row.
// With tpu_v > 0 the number of valid parts of a row follows from the work decomposition.
__global__ void combine_kernel(const float* __restrict__ parts, int n_parts, int64_t rows, int d, int out_dtype,
                               void* __restrict__ out, int64_t os_b, int64_t os_h, int64_t os_t, int Hq, int Tq, int G,
                               int B, int tpu_v, int L, int nw, float* __restrict__ merged,
                               const uint32_t* __restrict__ status, uint32_t epoch, int part_major) {
  const int64_t row = blockIdx.x;
  if (row >= rows) return;
  const bool failed = status != nullptr && *status == epoch;   // the attention kernel gave up on a wait
  const int64_t tq = row % Tq, bh = row / Tq, hq = bh % Hq, b = bh / Hq;
  int n_valid = n_parts;
  if (tpu_v > 0) {
    const int64_t u = (hq / G) * (int64_t)(B * Tq) + b * Tq + tq;
    const int64_t c0 = (u * tpu_v) / L, c1 = ((u + 1) * tpu_v - 1) / L;
    n_valid = (int)(c1 - c0 + 1) * nw;
  }
  // part i of this row: [row][i] (row-major parts) or [i][row] (one block of rows per part, as gathered from ranks)
  const float* base = part_major ? parts + row * (d + 2) : parts + row * n_parts * (d + 2);
  const int64_t ps = part_major ? rows * (int64_t)(d + 2) : (int64_t)(d + 2);
  // weights of the parts, computed once by the block: w_i = 2^(m_i - m*)
  extern __shared__ float s_w[];          // [n_valid]
  __shared__ float s_red[32];
  float m_loc = -INFINITY;
  for (int i = threadIdx.x; i < n_valid; i += blockDim.x) m_loc = fmaxf(m_loc, base[i * ps + d]);
  for (int o = 16; o > 0; o >>= 1) m_loc = fmaxf(m_loc, __shfl_xor_sync(0xffffffffu, m_loc, o));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m_loc;
  __syncthreads();
  float m_star = -INFINITY;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) m_star = fmaxf(m_star, s_red[i]);
  __syncthreads();
  const float m_use = m_star == -INFINITY ? 0.f : m_star;
  float l_loc = 0.f;
  for (int i = threadIdx.x; i < n_valid; i += blockDim.x) {
    const float w = exp2f(base[i * ps + d] - m_use);
    s_w[i] = w;
    l_loc += base[i * ps + d + 1] * w;
  }
  for (int o = 16; o > 0; o >>= 1) l_loc += __shfl_xor_sync(0xffffffffu, l_loc, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = l_loc;
  __syncthreads();
  float l_star = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) l_star += s_red[i];
  for (int x = threadIdx.x; x < d; x += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < n_valid; ++i) {
      const float w = s_w[i];
      if (w != 0.f) acc += base[i * ps + x] * w;
    }
    if (failed) acc = NAN;
    if (merged) merged[row * (d + 2) + x] = acc;
    else store_float(out, b * os_b + hq * os_h + tq * os_t + x, l_star > 0.f || failed ? acc / l_star : 0.f, out_dtype);
  }
  if (merged && threadIdx.x == 0) { merged[row * (d + 2) + d] = m_star; merged[row * (d + 2) + d + 1] = l_star; }
}

struct Plan {
  const void* kernel;
  size_t smem;
  int table_rows, ib, nw, rep_log2;
  int threads;                             // threads per CTA (the ring kernels add a producer warp to their nw consumers)
  int repv_log2, ring_stages, merge_slots; // ring kernels only
  size_t ticket_bytes;                     // ring kernels: one ticket word per unit between the status word and the partials
  int ppc;   // partials a CTA writes per unit and head: 1 for the staged kernels (merged in shared memory), nw otherwise
  int warp_units;   // staged kernels: warp mode (the warps walk through the units independently; ppc = nw)
  int units, tpu_v, L, P, grid;
  size_t ws_bytes;
};

static int validate_attn(const hqmq_attn_args* a) {
  if (!a || a->struct_size != sizeof(hqmq_attn_args)) return HQMQ_ERR_ARG;
  if (!a->Q || (!a->O && !a->partials_only)) return HQMQ_ERR_ARG;
  if (!is_float_dtype(a->q_dtype) || !is_float_dtype(a->o_dtype)) return HQMQ_ERR_DTYPE;
  if (a->B < 1 || a->H_q < 1 || a->H_kv < 1 || a->T_q < 1 || a->T_kv < 0 || a->d < 1) return HQMQ_ERR_SHAPE;
  if (a->H_q % a->H_kv) return HQMQ_ERR_SHAPE;
  if (a->H_q / a->H_kv > 16) return HQMQ_ERR_UNSUPPORTED;
  if (a->d % 16) return HQMQ_ERR_SHAPE;
  const int n = a->d / 4;
  if (!(n == 4 || n == 8 || n == 12 || n == 16 || n == 32)) return HQMQ_ERR_UNSUPPORTED;
  if (a->r_qmax < 1 || a->r_qmax > 1023) return HQMQ_ERR_SHAPE;
  if (a->partials_only && !a->partials) return HQMQ_ERR_ARG;
  if (a->kv_splits < 0 || a->window < 0 || a->causal < 0 || a->causal > 2) return HQMQ_ERR_ARG;
  if (a->layout == 0) {
    int rc = check_packed(a->K, false);
    if (rc) return rc;
    rc = check_packed(a->V, false);
    if (rc) return rc;
    if (a->K.B != a->B || a->V.B != a->B || a->K.H != a->H_kv || a->V.H != a->H_kv) return HQMQ_ERR_SHAPE;
    if (a->K.n_chunks != n || a->V.n_chunks != n) return HQMQ_ERR_SHAPE;
    if (a->K.S != a->V.S || a->K.radius_bits != a->V.radius_bits || a->K.scale_dtype != a->V.scale_dtype)
      return HQMQ_ERR_UNSUPPORTED;
    if (a->r_qmax != (1 << a->K.radius_bits) - 1) return HQMQ_ERR_SHAPE;
    if (a->T_kv > a->K.T_cap || a->T_kv > a->V.T_cap) return HQMQ_ERR_CAPACITY;
    if (!a->table_K || !a->table_V) return HQMQ_ERR_ARG;
    if (((uintptr_t)a->table_K & 7) || ((uintptr_t)a->table_V & 7)) return HQMQ_ERR_ALIGN;
  } else if (a->layout == 1) {
    if (a->K_ref.struct_size != sizeof(hqmq_ref_packed) || a->V_ref.struct_size != sizeof(hqmq_ref_packed)) return HQMQ_ERR_ARG;
    if (!a->K_ref.idx || !a->K_ref.rq || !a->K_ref.rs || !a->V_ref.idx || !a->V_ref.rq || !a->V_ref.rs) return HQMQ_ERR_ARG;
    if (!a->joint_K || !a->joint_V || !is_float_dtype(a->joint_dtype)) return HQMQ_ERR_ARG;
    if (a->K_size < 1 || a->K_size > 65536) return HQMQ_ERR_SHAPE;
  } else {
    return HQMQ_ERR_ARG;
  }
  return HQMQ_OK;
}

// Resident CTAs of `kernel` on the current device (cached per kernel, shared-memory size and device).  The first
// query of a (kernel, size, device) also raises the kernel's dynamic shared-memory limit, so a launch never has to.
// Guarded by a mutex: host threads that serve different GPUs call into the library concurrently.
static int resident_ctas(const void* kernel, size_t smem, int threads) {
  struct Entry { const void* k; size_t smem; int dev; int val; };
  static Entry cache[128];
  static int n_cache = 0;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_cache; ++i)
    if (cache[i].k == kernel && cache[i].smem == smem && cache[i].dev == dev) return cache[i].val;
  int sms = 0, occ = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // The limit is set to the device's opt-in maximum, not to this size: one kernel runs with several shared-memory
  // sizes (replication and warp mode depend on the problem), and a limit set to a later, smaller size would fail the
  // launch of an earlier size whose cached answer skips this step.
  if (smem > 48 * 1024) {
    int optin = 0;
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, optin > (int)smem ? optin : (int)smem);
  }
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, smem) != cudaSuccess || occ < 1) occ = 1;
  cudaGetLastError();
  const int val = (sms > 0 ? sms : 148) * occ;
  if (n_cache < 128) cache[n_cache++] = {kernel, smem, dev, val};
  return val;
}

// Units of at most this many tiles run the staged kernels in warp mode (every warp has at most two tiles of a unit)
constexpr int kWarpModeMaxTiles = 32;

static int make_plan_impl(const hqmq_attn_args* a, Plan& pl, bool query_device, bool allow_warp_mode) {
  const int n = a->d / 4;
  const int G = a->H_q / a->H_kv;
  const bool outl = a->layout == 0 && (a->K.flags != nullptr || a->V.flags != nullptr);
  pl.kernel = nullptr;
  pl.nw = kSlowWarps;
  pl.rep_log2 = 0;
  if (a->layout == 0) {
    pl.ib = idx_bits_for(a->K.S);
    pl.table_rows = 24 * a->K.S;
    // the staged kernels copy 16-byte aligned pieces: side buffers must start on 16 bytes per (b,h)
    const bool side_ok = !outl || (((!a->K.flags || (a->K.out_cap % 2 == 0 && ((uintptr_t)a->K.out_vals & 15) == 0))) &&
                                   ((!a->V.flags || (a->V.out_cap % 2 == 0 && ((uintptr_t)a->V.out_vals & 15) == 0))));
    if (G <= 8 && is_half_dtype(a->K.scale_dtype) && side_ok) pl.kernel = fast_kernel(n, pl.ib, a->K.radius_bits, outl);
    if (pl.kernel) pl.nw = outl ? kFastWarpsOutl : kFastWarps;
  } else {
    pl.ib = 16;
    pl.table_rows = a->K_size;
  }
  const bool fast = pl.kernel != nullptr;
  pl.ppc = fast ? 1 : kSlowWarps;
  if (!pl.kernel) pl.kernel = slow_kernel(n, outl, G > 8);
  if (!pl.kernel) return HQMQ_ERR_UNSUPPORTED;
  pl.threads = pl.nw * 32;
  pl.repv_log2 = pl.ring_stages = pl.merge_slots = 0;
  const int keys = a->window > 0 ? (a->window < a->T_kv ? a->window : a->T_kv) : a->T_kv;
  // Long key ranges: the kernels with one CTA-wide staging ring.  The kernels are bound by shared-memory bandwidth
  // (the random 8-byte codeword gathers), so shared memory goes first to the replication of the sign-folded tables
  // (K at least as much as V) next to a two-stage ring, then to a third stage, then to merge slots (measured: a
  // third stage bought nothing where it cost a table replica).
  RingKernelInfo rk;
  bool ring = false;
  const int64_t tiles_all = (int64_t)a->B * a->T_q * a->H_kv * ((keys + kTile - 1) / kTile);
  if (fast && keys >= kRingMinKeys && tiles_all >= kRingMinTiles && ring_kernel(n, pl.ib, a->K.radius_bits, outl, a->K.scale_dtype, rk)) {
    auto fits = [&](int rsum, int ns, int ms) {
      return ring_smem_total(pl.table_rows, (rsum + 1) / 2, rsum / 2, a->d, outl, ns, ms, rk.stage_bytes, rk.warps) <= kSmemLimit;
    };
    if (fits(0, 2, 1)) {
      int rsum = 0;
      while (rsum < 8 && fits(rsum + 1, 2, 1)) ++rsum;
      ring = true;
      pl.rep_log2 = (rsum + 1) / 2; pl.repv_log2 = rsum / 2; pl.ring_stages = 2; pl.merge_slots = 1;
      while (pl.ring_stages < 4 && fits(rsum, pl.ring_stages + 1, 1)) ++pl.ring_stages;
      // The d_head-64 kernels (19 consumer warps, bigger stages, a tile that is done sooner) run out of staged tiles
      // with two stages: there the last replica of V goes to a third stage instead (measured on a B64 x 16384-token
      // layer: 463 -> 437 us; at d_head 128 a third stage bought nothing where it cost a replica).
      if (rk.warps > 15 && pl.ring_stages < 3 && rsum > 0 && fits(rsum - 1, 3, 1)) {
        --rsum;
        pl.rep_log2 = (rsum + 1) / 2; pl.repv_log2 = rsum / 2; pl.ring_stages = 3;
      }
      for (int ms : {5, 3})
        if (fits(rsum, pl.ring_stages, ms)) { pl.merge_slots = ms; break; }
    }
  }
  // tiles a unit can have (a window may straddle one extra tile)
  int tpu = (keys + kTile - 1) / kTile + (a->window > 0 ? 1 : 0);
  if (tpu < 1) tpu = 1;
  pl.units = a->B * a->T_q * a->H_kv;
  // Staged kernels, many short units: warp mode.  Every warp then writes its own partial per unit and CTA (16 times
  // the scratch of the in-CTA merge), so a caller whose scratch is fixed can rule it out.
  {
    // (a CTA's piece of the flat tile sequence: at least a tile per warp; warp mode pays when it spans several units)
    const int64_t piece = std::max<int64_t>(((int64_t)pl.units * tpu + 147) / 148, pl.nw);
    pl.warp_units = fast && !ring && allow_warp_mode && a->kv_splits == 0 && tpu <= kWarpModeMaxTiles && tpu < piece;
  }
  if (pl.warp_units) pl.ppc = pl.nw;
  if (ring) {
    pl.kernel = rk.fn;
    pl.nw = rk.warps;
    pl.threads = (rk.warps + 1) * 32;
    pl.smem = ring_smem_total(pl.table_rows, pl.rep_log2, pl.repv_log2, a->d, outl, pl.ring_stages, pl.merge_slots, rk.stage_bytes, rk.warps);
  } else {
  const int nheads = G > 8 ? 16 : 8;
  size_t extra = outl ? (size_t)nheads * a->d * 4 + (size_t)pl.nw * (2 * kStage * 8 + 16 * nheads * 4) : 0;
  if (fast)
    extra = (outl ? (size_t)(pl.warp_units ? pl.nw : 1) * 8 * (a->d + kFastQPad) * 2 : 0) + (((size_t)pl.nw * kFastStages * 8 + 15) & ~(size_t)15) +
            (size_t)pl.nw * fast_warp_bytes(n, pl.ib, a->K.radius_bits, outl);
  // The big-CTA kernels own a whole SM: replicate the tables (interleaved) as far as shared memory
  // allows, which spreads the random codeword gathers over more banks.
  // bytes of both tables without replication (the staged kernels keep sign-folded, half-size tables)
  const size_t tbl_unit = (fast && !outl) ? (size_t)pl.table_rows * 8 : (size_t)pl.table_rows * 16;
  if (fast)
    while (pl.rep_log2 < 4 && (tbl_unit << (pl.rep_log2 + 1)) + extra <= 224 * 1024) ++pl.rep_log2;
  pl.smem = (tbl_unit << pl.rep_log2) + extra;
  if (pl.smem > kSmemLimit) {
    if (!fast) return HQMQ_ERR_UNSUPPORTED;
    // the staged kernel does not fit next to this codebook: use the generic one
    pl.kernel = slow_kernel(n, outl, false);
    pl.nw = kSlowWarps; pl.rep_log2 = 0; pl.ppc = kSlowWarps; pl.warp_units = 0;
    pl.threads = pl.nw * 32;
    pl.smem = (size_t)pl.table_rows * 16 + (outl ? (size_t)8 * a->d * 4 + (size_t)pl.nw * (2 * kStage * 8 + 16 * 8 * 4) : 0);
    if (pl.smem > kSmemLimit) return HQMQ_ERR_UNSUPPORTED;
  }
  }

  // (asked on every path: the first query of a kernel also raises its dynamic shared-memory limit)
  int slots = query_device ? resident_ctas(pl.kernel, pl.smem, pl.threads) : 148;
  if (slots < 1) slots = 1;
  if (a->kv_splits > 0) {
    int splits = a->kv_splits < tpu ? a->kv_splits : tpu;
    pl.L = (tpu + splits - 1) / splits;
    pl.tpu_v = pl.L * splits;
  } else {
    // equal pieces of the flat tile sequence, one per resident CTA; at least one tile per warp
    pl.tpu_v = tpu;
    const int64_t total = (int64_t)pl.units * tpu;
    int64_t L = (total + slots - 1) / slots;
    if (L < pl.nw) L = pl.nw;
    if (L > total) L = total;
    pl.L = (int)L;
  }
  const int64_t total = (int64_t)pl.units * pl.tpu_v;
  pl.grid = (int)((total + pl.L - 1) / pl.L);
  pl.P = (pl.tpu_v - 1 + pl.L - 1) / pl.L + 1;
  // Ring kernels with fewer units than CTAs: CTA boundaries snapped to unit boundaries when that is cheaper than the
  // flat split, whose straddling CTAs pay a second unit's set-up and merge -- about 80 tiles' worth of time, 130 when
  // the next unit is another KV head and the tables are reloaded (one sequence of 131072 tokens: the 7 straddling CTAs
  // finished at 138 us, the other 141 at 105).  Every unit is cut into c = slots / units equal pieces of Lu tiles; in
  // the kernel's terms that is a flat split of L = Lu over units of c * Lu virtual tiles (the tiles past a unit's real
  // ones are empty), so the kernel needs no other code for it.
  if (pl.ring_stages > 0 && a->kv_splits == 0 && pl.units < slots) {
    const int c = slots / pl.units;
    const int Lu = (tpu + c - 1) / c;
    const int straddle = a->B * a->T_q == 1 ? 130 : 80;
    if (pl.L < tpu && Lu >= pl.nw && Lu < pl.L + straddle) {
      pl.L = Lu;
      pl.tpu_v = c * Lu;
      pl.grid = pl.units * c;
      pl.P = c;
    }
  }
  const int64_t rows = (int64_t)a->B * a->H_q * a->T_q;
  pl.ticket_bytes = pl.ring_stages ? (((size_t)pl.units * 4 + 15) & ~(size_t)15) : 0;
  pl.ws_bytes = 16 + pl.ticket_bytes + (size_t)rows * pl.P * pl.ppc * (a->d + 2) * sizeof(float);
  return HQMQ_OK;
}

// Warp mode is dropped where its scratch (a partial per warp instead of one per CTA) would pass kWarpModeMaxScratch.
constexpr size_t kWarpModeMaxScratch = (size_t)256 << 20;
static int make_plan(const hqmq_attn_args* a, Plan& pl, bool query_device, bool allow_warp_mode = true) {
  int rc = make_plan_impl(a, pl, query_device, allow_warp_mode);
  if (rc == HQMQ_OK && pl.warp_units && pl.ws_bytes > kWarpModeMaxScratch) rc = make_plan_impl(a, pl, query_device, false);
  return rc;
}

// The workspace must not depend on the device's occupancy answer changing between the size query
// and the call; both use the same plan, and the size is an upper bound over L >= the planned one.
}  // namespace attn
}  // namespace hqmq

using namespace hqmq;
using namespace hqmq::attn;

extern "C" size_t hqmq_attn_workspace_bytes(const hqmq_attn_args* a) {
  if (validate_attn(a) != HQMQ_OK) return 0;
  Plan pl;
  if (make_plan(a, pl, true) != HQMQ_OK) return 0;
  return pl.ws_bytes;
}

extern "C" int hqmq_combine_partials(const float* parts, int n_parts, int64_t rows, int d, int part_major, int out_dtype,
                                     void* out, void* stream) {
  if (!parts || !out) return HQMQ_ERR_ARG;
  if (n_parts < 1 || rows < 0 || d < 1) return HQMQ_ERR_SHAPE;
  if (!is_float_dtype(out_dtype)) return HQMQ_ERR_DTYPE;
  if (rows == 0) return HQMQ_OK;
  // rows are laid out contiguously: treat as B = rows, Hq = Tq = 1
  combine_kernel<<<(unsigned)rows, 128, (size_t)n_parts * 4, (cudaStream_t)stream>>>(parts, n_parts, rows, d, out_dtype, out, d, 0, 0, 1, 1, 1,
                                                                  (int)rows, 0, 1, 1, nullptr, nullptr, 0u, part_major ? 1 : 0);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

extern "C" int hqmq_attn_decode(const hqmq_attn_args* a, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = validate_attn(a);
  if (rc) return rc;
  Plan pl;
  rc = make_plan(a, pl, true);
  if (rc) return rc;
  if (workspace && workspace_bytes < pl.ws_bytes && pl.warp_units) {
    // a scratch sized for the in-CTA merge (the built-in one of hqmq_attn_decode_static): plan without warp mode
    rc = make_plan(a, pl, true, false);
    if (rc) return rc;
  }
  if (!workspace || workspace_bytes < pl.ws_bytes) return HQMQ_ERR_WORKSPACE;
  if ((uintptr_t)workspace & 15) return HQMQ_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;

  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.B = a->B; p.Hq = a->H_q; p.Hkv = a->H_kv; p.G = a->H_q / a->H_kv; p.Tq = a->T_q; p.Tkv = a->T_kv; p.d = a->d;
  p.causal = a->causal; p.window = a->window;
  const float scale = a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / sqrtf((float)a->d);
  p.sscale = scale * 1.4426950408889634f / (float)a->r_qmax;
  p.qscale = scale * 1.4426950408889634f;
  p.nw = pl.nw; p.rep_log2 = pl.rep_log2; p.warp_units = pl.warp_units;
  // (ring kernels of d_head 64 with two or more units per CTA: the units of a CTA are taken from different KV heads)
  p.unit_hfast = pl.ring_stages > 0 && a->d == 64 && a->H_kv > 1 && pl.units >= 2 * pl.grid;
  p.repv_log2 = pl.repv_log2; p.ring_stages = pl.ring_stages; p.merge_slots = pl.merge_slots;
  p.vscale = 1.0f / (float)a->r_qmax;
  p.qmaxf = (float)a->r_qmax;
  p.units = pl.units; p.tpu_v = pl.tpu_v; p.L = pl.L; p.P = pl.P;
  p.Q = a->Q; p.q_dtype = a->q_dtype; p.qs_b = a->q_stride[0]; p.qs_h = a->q_stride[1]; p.qs_t = a->q_stride[2];
  static std::atomic<uint32_t> epoch_counter{0x5eed0000u};
  p.status = reinterpret_cast<uint32_t*>(workspace);
  p.epoch = epoch_counter.fetch_add(1u, std::memory_order_relaxed) + 1u;
  p.tickets = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(workspace) + 16);
  p.partials = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + 16 + pl.ticket_bytes);
  p.O = a->O; p.o_dtype = a->o_dtype; p.os_b = a->o_stride[0]; p.os_h = a->o_stride[1]; p.os_t = a->o_stride[2];
  p.merged = a->partials_only ? a->partials : nullptr;
  const bool fused_merge = pl.ring_stages > 0;   // the ring kernels merge a unit's partials themselves (last CTA of the unit)
  if (fused_merge) HQMQ_CHECK_CUDA(cudaMemsetAsync(p.tickets, 0, pl.ticket_bytes, st));
  p.layout = a->layout;
  p.table_rows = pl.table_rows;
  p.ib = pl.ib;
  if (a->layout == 0) {
    p.K = a->K; p.V = a->V; p.tblK = a->table_K; p.tblV = a->table_V;
  } else {
    p.Kr = a->K_ref; p.Vr = a->V_ref; p.jK = a->joint_K; p.jV = a->joint_V; p.j_dtype = a->joint_dtype;
  }
  // (the kernel's dynamic shared-memory limit was raised when the plan asked for its occupancy: resident_ctas)
  void* kargs[] = {&p};
  HQMQ_CHECK_CUDA(cudaLaunchKernel(pl.kernel, dim3(pl.grid), dim3(pl.threads), kargs, pl.smem, st));
  if (fused_merge) { HQMQ_LAUNCH_CHECK(); return HQMQ_OK; }
  const int64_t rows = (int64_t)a->B * a->H_q * a->T_q;
  combine_kernel<<<(unsigned)rows, a->d < 128 ? 64 : 128, (size_t)pl.P * pl.ppc * 4, st>>>(
      p.partials, pl.P * pl.ppc, rows, a->d, a->o_dtype, a->O, a->o_stride[0], a->o_stride[1], a->o_stride[2], a->H_q,
      a->T_q, p.G, a->B, pl.tpu_v, pl.L, pl.ppc, a->partials_only ? a->partials : nullptr, p.status, p.epoch, 0);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}


// ---- decode attention without any allocation by anybody ---------------------------------------------------
// Some hosts cannot hand this library a workspace: a serving process that gave every free byte of HBM to its
// KV-cache pool at start-up (so a later cudaMalloc fails), or a thin foreign-language binding that exposes no
// device allocator at all.  For them the partials of hqmq_attn_decode live in a buffer that is part of the
// library image: every GPU that loads the library holds HQMQ_ATTN_STATIC_SCRATCH_BYTES of it until the process
// exits.  The array's name is only a host-side handle, so its device address is looked up once per device
// (with that device current) and cached.
namespace {
__device__ __align__(256) unsigned char g_attn_static_scratch[HQMQ_ATTN_STATIC_SCRATCH_BYTES];
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};
}  // namespace

extern "C" int hqmq_attn_decode_static(const hqmq_attn_args* a, void* stream) {
  int rc = validate_attn(a);
  if (rc) return rc;
  Plan pl;
  rc = make_plan(a, pl, true);
  if (rc) return rc;
  if (pl.ws_bytes > (size_t)HQMQ_ATTN_STATIC_SCRATCH_BYTES && pl.warp_units) {
    rc = make_plan(a, pl, true, false);   // (hqmq_attn_decode below makes the same choice from the size it is given)
    if (rc) return rc;
  }
  if (pl.ws_bytes > (size_t)HQMQ_ATTN_STATIC_SCRATCH_BYTES) return HQMQ_ERR_STATIC_SCRATCH;
  int dev = -1;
  HQMQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return HQMQ_ERR_UNSUPPORTED;
  void* ptr = __atomic_load_n(&g_static_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (!ptr) {
    // first call on this device: resolve the device address of the array (racing first calls resolve
    // the same address, so the last store wins harmlessly)
    if (cudaGetSymbolAddress(&ptr, g_attn_static_scratch) != cudaSuccess || !ptr) return HQMQ_ERR_CUDA;
    __atomic_store_n(&g_static_scratch_ptr[dev], ptr, __ATOMIC_RELEASE);
  }
  // Of everything in the scratch only the give-up word has to start at zero: every partial that is read was
  // written by this call.  The word is cleared on the stream ahead of the kernels, so that after the call it
  // tells about this call alone (also when the call is replayed from a captured graph with its epoch baked in).
  HQMQ_CHECK_CUDA(cudaMemsetAsync(ptr, 0, 16, (cudaStream_t)stream));
  return hqmq_attn_decode(a, ptr, (size_t)HQMQ_ATTN_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int hqmq_attn_static_status(uint32_t* status, void* stream) {
  if (!status) return HQMQ_ERR_ARG;
  int dev = -1;
  HQMQ_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return HQMQ_ERR_UNSUPPORTED;
  void* ptr = __atomic_load_n(&g_static_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (!ptr) { *status = 0; return HQMQ_OK; }   // no static call was made on this device yet
  return hqmq_read_status(ptr, status, stream);
}
