// Decode attention over the native compressed cache, long key ranges: one CTA per SM with ONE staging ring
// shared by all of its warps.
//
//   producer   one extra warp.  A stage of the ring holds one 16-token tile per consumer warp, consecutive tiles of
//              a unit (240 or 304 tokens): the code rows of K and V, the two scale vectors and, with Med3x, the flag words,
//              the tiles' slices of the outlier side buffers and the K fragment records.  A stage is a handful
//              of bulk asynchronous copies (cp.async.bulk, 8-20 KB each) that complete on the stage's "full"
//              mbarrier, so the cost of issuing copies is shared by all tiles of the stage.
//   consumers  ring_warps(chunks per token) warps; warp w decodes tile w of every stage, then arrives on the stage's "empty"
//              mbarrier, which lets the producer refill the buffer.
// The codeword tables are SIGN-FOLDED (only the even native indices are kept, the sign of the axis unit goes
// into the radius) and replicated 2^r times, interleaved entry by entry: random 8-byte gathers cost 5.0 / 4.6 /
// 3.8 / 2.8 shared-memory cycles per warp at 1 / 4 / 8 / 16 replicas (measured), so K and V each get as many
// replicas as shared memory allows.
// Outliers: a tile of K that owns fragment records adds them with one shared-memory load and one MMA per
// record; every other flagged chunk (K tiles without records, all of V) is corrected in fp32 on the CUDA cores,
// one warp-wide step per flagged chunk, from the staged payload slice: its decoded value is 0 (radius code 0),
// so the correction is purely additive.  V tiles of d_head 64 whose flagged chunks fill a few chunk columns (an
// outlier channel) add them column by column with two MMAs each instead.
// The arithmetic of the tile (fragment layouts, online softmax) is the one described in attn_kernel.cuh.
#pragma once
#include "attn_tma.cuh"

namespace hqmq {
namespace attn {

// Consumer warps of a CTA (one more warp produces).  d_head 128: 15, with the producer 512 threads of 128 registers.
// d_head 64: a tile keeps half the accumulators and fields and fits 96 registers, so 19 consumers (640 threads, five
// warps per scheduler instead of four) hide more of the latencies of a tile whose fixed work -- softmax, headers,
// outlier columns -- is spread over half the bytes (measured on a B64 x 16384-token layer: 500 -> 458 us).
__host__ __device__ constexpr int ring_warps(int n_chunks) { return n_chunks == 16 ? 19 : 15; }

template <int N, int IB, int RB, bool OUTL>
struct RingLayout {
  static constexpr int W = ring_warps(N);        // tiles per stage: one per consumer warp
  static constexpr int kTok = W * kTile;         // tokens per stage
  static constexpr int kRec = W + 1;             // fragment records staged per stage
  static constexpr int ROW = N * (IB + RB) / 8;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTok * ROW;
  static constexpr int kRsK = kV + kTok * ROW;
  static constexpr int kRsV = kRsK + kTok * 2;
  static constexpr int kPlainEnd = kRsV + kTok * 2;
  static constexpr int kFlK = kPlainEnd;
  static constexpr int kFlV = kFlK + kTok * 4;
  static constexpr int kStageHdr = kFlV + kTok * 4;          // 32 bytes: what the producer staged
  static constexpr int kTileHdr = kStageHdr + 32;                // W x 32 bytes: the tiles' side ranges
  static constexpr int kPayV = kTileHdr + W * 32;
  // payload entries staged per stage and tensor (+2 alignment slack): d_head 64 has room for a stage whose every token
  // owns a flagged chunk (one outlier channel per head: an entry per token)
  static constexpr int kPay = N == 16 ? (W * kTile + 14) : 126;
  static constexpr int kSideK = kPayV + (kPay + 2) * 8;      // K payload slice, or the stage's fragment records
  static constexpr int kSideKBytes = kRec * HQMQ_OFRAG_BYTES > (kPay + 2) * 8 ? kRec * HQMQ_OFRAG_BYTES
                                                                                    : (kPay + 2) * 8;
  static constexpr int BYTES = OUTL ? kSideK + kSideKBytes : kPlainEnd;
  static_assert((kTok * ROW) % 16 == 0 && (kTok * 2) % 16 == 0 && BYTES % 16 == 0, "stage pieces must be multiples of 16 bytes");
};

// What the host must know about the kernel's shared memory (the device derives the same offsets).
struct RingSmem {
  size_t tblK, tblV, q, bars, merge, ring, total;
};
__host__ __device__ inline RingSmem ring_smem(int table_rows, int repk_log2, int repv_log2, int d, bool outl, int stages,
                                               int merge_slots, size_t stage_bytes, int warps) {
  RingSmem s;
  size_t o = 0;
  s.tblK = o; o += (size_t)(table_rows >> 1) * (8u << repk_log2);
  s.tblV = o; o += (size_t)(table_rows >> 1) * (8u << repv_log2);
  s.q = o; o += outl ? (size_t)8 * (d + kQPad) * 2 : 0;
  o = (o + 15) & ~(size_t)15;
  s.bars = o; o += 64;                                   // full[4], empty[4]
  // merge area: m[warps][8], l[warps][8], weight[warps][8], m*[8], l*[8], abort word, then `merge_slots` slots of [8][d] floats
  s.merge = o; o += (size_t)(3 * warps * 8 + 16 + 4) * 4 + (size_t)merge_slots * 8 * d * 4;
  o = (o + 127) & ~(size_t)127;
  s.ring = o; o += (size_t)stages * stage_bytes;
  s.total = o;
  return s;
}

__device__ __forceinline__ float rcp_fast(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
template <int THREADS>
__device__ __forceinline__ void consumer_bar_n() {
  asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}
// Barrier among the consumer threads that also ORs a predicate over them.
template <int THREADS>
__device__ __forceinline__ bool consumer_bar_or_n(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.u32 p, %1, 0;\n barrier.cta.red.or.pred q, 1, %2, p;\n selp.u32 %0, 1, 0, q;\n}\n"
      : "=r"(r) : "r"((uint32_t)pred), "n"(THREADS) : "memory");
  return r != 0;
}

// The piece of unit u that belongs to this CTA: tiles [my_lo, my_hi) and the CTA's slot among the unit's CTAs.
struct UnitPiece { int h, b, tq, t_beg, t_end, my_lo, my_hi, part; };
// HFAST: the kernel honours p.unit_hfast -- units numbered with the KV head running fastest, u = (b, tq) * H_kv + h, so
// that the units of one CTA belong to different heads.  Heads differ in outlier density (an outlier channel flags a
// chunk in every token of one head and hardly any of another), and with equal tile counts the CTAs of the dense heads
// set the kernel's time: B64 x 8 heads x 16384 tokens at d_head 64, 3.5 units per CTA, 444 -> 419 us for a table
// reload at every unit boundary.  (The d_head 128 kernels keep the head-major order: their CTAs hold at most two units
// in the configurations measured, and the order made no difference there.)
template <bool HFAST>
__device__ __forceinline__ UnitPiece unit_piece(const AttnParams& p, int u, int64_t flat_lo, int64_t flat_hi) {
  UnitPiece q;
  const int upb = p.B * p.Tq;
  int bt;
  if (HFAST && p.unit_hfast) { bt = u / p.Hkv; q.h = u - bt * p.Hkv; }
  else { q.h = u / upb; bt = u - q.h * upb; }
  q.b = bt / p.Tq; q.tq = bt - q.b * p.Tq;
  key_range(p.Tkv, p.Tq, p.causal, p.window, q.tq, q.t_beg, q.t_end);
  const int tile_lo = q.t_beg / kTile, tile_hi = (q.t_end + kTile - 1) / kTile;
  const int64_t ubase = (int64_t)u * p.tpu_v;
  const int rel_lo = (int)(flat_lo > ubase ? flat_lo - ubase : 0);
  const int rel_hi = (int)(flat_hi < ubase + p.tpu_v ? flat_hi - ubase : p.tpu_v);
  q.my_lo = tile_lo + rel_lo;
  q.my_hi = min(tile_hi, tile_lo + rel_hi);
  q.part = (int)blockIdx.x - (int)(ubase / p.L);
  return q;
}

// Bounded wait on an mbarrier phase.  Each try may suspend the thread in hardware for up to kRingSuspendNs (it is
// woken as soon as the phase completes), so a waiting warp costs a handful of instructions instead of a spin loop;
// kRingWaitTries of them bound the wait to about a second.  Gives up early when another warp already gave up.
constexpr uint32_t kRingSuspendNs = 10u * 1000u * 1000u;
constexpr uint32_t kRingWaitTries = 100u;
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(kRingSuspendNs) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_word) {
  uint32_t tries = 0;
  while (!mbar_try_wait_suspend(bar, parity)) {
    if (++tries > kRingWaitTries || *abort_word) return false;
  }
  return true;
}

// The producer's wait for a released buffer.  It has a whole stage of slack (the consumers work on the other buffers
// meanwhile), so it tests the barrier without blocking and sleeps between tests: a waiting producer then costs
// the consumers neither issue slots nor shared-memory cycles.  Bounded like ring_wait (about a second).
constexpr uint32_t kProducerSleepNs = 160u;
constexpr uint32_t kProducerTries = 6u * 1000u * 1000u;
__device__ __forceinline__ bool ring_wait_producer(uint32_t bar, uint32_t parity, volatile uint32_t* abort_word) {
  uint32_t tries = 0;
  for (;;) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if (++tries > kProducerTries || *abort_word) return false;
    __nanosleep(kProducerSleepNs);
  }
}

template <int N, int IB, int RB, bool OUTL, int SDT>
__device__ __forceinline__ void attn_ring_body(const AttnParams& p) {
  using G_ = Geo<N>;
  using FL = FastLoader<N, IB, RB, true>;
  using RL = RingLayout<N, IB, RB, OUTL>;
  constexpr int NKS = G_::NKS, NVG = G_::NVG, NOT = 2 * G_::NVG;
  constexpr int ROW = RL::ROW;
  constexpr int D = 4 * N;
  constexpr int kRingWarps = RL::W, kRingTiles = RL::W, kRingRec = RL::kRec, kRingConsumerThreads = RL::W * 32;
  auto consumer_bar = [] { consumer_bar_n<kRingConsumerThreads>(); };
  auto consumer_bar_or = [](bool pred) { return consumer_bar_or_n<kRingConsumerThreads>(pred); };
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int NS = p.ring_stages;
  const RingSmem sl = ring_smem(p.table_rows, p.rep_log2, p.repv_log2, p.d, OUTL, NS, p.merge_slots, RL::BYTES, kRingWarps);
  unsigned char* tblK = smem_raw + sl.tblK;
  unsigned char* tblV = smem_raw + sl.tblV;
  __half* qh16 = reinterpret_cast<__half*>(smem_raw + sl.q);
  constexpr int qstride = D + kQPad;
  const uint32_t bar_full = smem_u32(smem_raw + sl.bars), bar_empty = bar_full + 32;
  float* m_s = reinterpret_cast<float*>(smem_raw + sl.merge);      // [16][8]
  float* l_s = m_s + kRingWarps * 8;                                // [16][8]
  float* w_s = l_s + kRingWarps * 8;                                // [16][8]
  float* ms_s = w_s + kRingWarps * 8;                               // [8] m*, [8] l*
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(ms_s + 16);
  volatile uint32_t* last_s = abort_word + 1;                       // "this CTA drew the unit's last ticket"
  float* slots = ms_s + 20;                                         // [merge_slots][8][D]
  unsigned char* ring = smem_raw + sl.ring;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, kRingWarps); }
    *abort_word = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int64_t flat_lo = (int64_t)blockIdx.x * p.L;
  const int64_t flat_total = (int64_t)p.units * p.tpu_v;
  const int64_t flat_hi = flat_lo + p.L < flat_total ? flat_lo + p.L : flat_total;
  const int u_first = (int)(flat_lo / p.tpu_v);

  // =============================== producer warp ==============================================================
  if (warp == kRingWarps) {
    uint32_t gs = 0;          // stages issued so far
    bool ok = true;
    const bool hasFlK = OUTL && p.K.flags != nullptr, hasFlV = OUTL && p.V.flags != nullptr;
    const bool stageK = hasFlK && p.K.out_dtype != HQMQ_F32, stageV = hasFlV && p.V.out_dtype != HQMQ_F32;
    const bool hasFr = hasFlK && p.K.ofrag != nullptr;
    // The stages of this CTA's piece, in order: (unit, first tile).  A unit without tiles in the piece has none.
    struct StageIt { int u, tile0; bool valid; UnitPiece up; };
    auto seek = [&](StageIt& it) {          // first unit from it.u on that has tiles here
      it.valid = false;
      for (; (int64_t)it.u * p.tpu_v < flat_hi; ++it.u) {
        it.up = unit_piece<N == 16>(p, it.u, flat_lo, flat_hi);
        if (it.up.my_lo < it.up.my_hi) { it.tile0 = it.up.my_lo; it.valid = true; break; }
      }
    };
    auto advance = [&](StageIt& it) {
      it.tile0 += kRingTiles;
      if (it.tile0 >= it.up.my_hi) { ++it.u; seek(it); }
    };
    // side ranges of a stage's tiles: lane l holds the offsets before tile l of the stage (l <= tiles of the stage)
    auto load_side = [&](const StageIt& it, uint32_t& kOff, uint32_t& vOff, uint32_t& fOff) {
      kOff = vOff = fOff = 0;
      if constexpr (OUTL) {
        if (it.valid) {
          const int nt_ = min(kRingTiles, it.up.my_hi - it.tile0);
          if (lane <= nt_) {
            const int64_t bh_ = (int64_t)it.up.b * p.Hkv + it.up.h;
            const int64_t nb = bh_ * (p.K.T_cap / HQMQ_OUT_BLOCK + 1) + it.tile0 + lane;
            if (hasFlK) kOff = p.K.out_off[nb];
            if (hasFr) fOff = p.K.ofrag_off[nb];
            if (hasFlV) vOff = p.V.out_off[bh_ * (p.V.T_cap / HQMQ_OUT_BLOCK + 1) + it.tile0 + lane];
          }
        }
      }
    };
    StageIt cur;
    cur.u = u_first;
    seek(cur);
    uint32_t kOff, vOff, fOff;
    load_side(cur, kOff, vOff, fOff);
    for (; ok && cur.valid; ++gs) {
      {
        const UnitPiece& up = cur.up;
        const int tile0 = cur.tile0;
        const int64_t bh = (int64_t)up.b * p.Hkv + up.h;
        const int nt = min(kRingTiles, up.my_hi - tile0);
        const int buf = gs % NS;
        unsigned char* sb = ring + (size_t)buf * RL::BYTES;
        // the next stage's side ranges are fetched now (global loads in flight across the wait and the issue below)
        StageIt nxt = cur;
        advance(nxt);
        uint32_t kOffN, vOffN, fOffN;
        load_side(nxt, kOffN, vOffN, fOffN);
        if (gs >= (uint32_t)NS) {
          ok = ring_wait(bar_empty + 8 * buf, ((gs / NS) - 1u) & 1u, abort_word);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        uint32_t bytes = 2u * nt * kTile * ROW + 2u * nt * kTile * 2;
        uint32_t ak = 0, nK = 0, av = 0, nV = 0, f0 = 0, nR = 0;
        bool flk = false, flv = false;
        if constexpr (OUTL) {
          const uint32_t kNext = __shfl_down_sync(0xffffffffu, kOff, 1), vNext = __shfl_down_sync(0xffffffffu, vOff, 1);
          const uint32_t fNext = __shfl_down_sync(0xffffffffu, fOff, 1);
          if (lane < nt)
            *reinterpret_cast<uint4*>(sb + RL::kTileHdr + lane * 32) = make_uint4(kOff, kNext, vOff, vNext),
            *reinterpret_cast<uint4*>(sb + RL::kTileHdr + lane * 32 + 16) = make_uint4(fOff, fNext, 0u, 0u);
          // a tile needs its K flag words and payload when it has flagged chunks but owns no record
          flk = __ballot_sync(0xffffffffu, lane < nt && kNext > kOff && fNext <= fOff) != 0u;
          const uint32_t k0s = __shfl_sync(0xffffffffu, kOff, 0), k1s = __shfl_sync(0xffffffffu, kOff, nt);
          const uint32_t v0s = __shfl_sync(0xffffffffu, vOff, 0), v1s = __shfl_sync(0xffffffffu, vOff, nt);
          const uint32_t f0s = __shfl_sync(0xffffffffu, fOff, 0), f1s = __shfl_sync(0xffffffffu, fOff, nt);
          flv = v1s > v0s;
          // (entries at or beyond out_cap were dropped by the encoder: nothing of them is copied, they read as 0)
          if (flk && stageK) {
            ak = k0s & ~1u;
            nK = k1s - ak; if (nK > (uint32_t)RL::kPay + 1u) nK = RL::kPay + 1;
            const uint32_t room = ak < (uint32_t)p.K.out_cap ? (uint32_t)p.K.out_cap - ak : 0u;
            if (nK > room) nK = room;
            nK = (nK + 1u) & ~1u;
          }
          if (flv && stageV) {
            av = v0s & ~1u;
            nV = v1s - av; if (nV > (uint32_t)RL::kPay + 1u) nV = RL::kPay + 1;
            const uint32_t room = av < (uint32_t)p.V.out_cap ? (uint32_t)p.V.out_cap - av : 0u;
            if (nV > room) nV = room;
            nV = (nV + 1u) & ~1u;
          }
          // records and the K payload slice share one area: records are staged only when no tile needs payload
          f0 = f0s;
          if (!flk || !stageK) { nR = f1s - f0s; if (nR > (uint32_t)kRingRec) nR = kRingRec; }
          if (lane == 0) {
            *reinterpret_cast<uint4*>(sb + RL::kStageHdr) = make_uint4(ak, nK, av, nV);
            *reinterpret_cast<uint4*>(sb + RL::kStageHdr + 16) = make_uint4(f0, nR, (flk ? 1u : 0u) | (flv ? 2u : 0u), 0u);
          }
          bytes += (flk ? nt * kTile * 4u : 0u) + (flv ? nt * kTile * 4u : 0u) + nK * 8u + nV * 8u + nR * HQMQ_OFRAG_BYTES;
          __syncwarp();    // the headers are written before lane 0's arrive publishes the stage
        }
        if (lane == 0) {
          const uint32_t sb32 = smem_u32(sb), bar = bar_full + 8 * buf;
          mbar_expect_tx(bar, bytes);
          const int64_t rowK = bh * p.K.T_cap + (int64_t)tile0 * kTile, rowV = bh * p.V.T_cap + (int64_t)tile0 * kTile;
          bulk_g2s(sb32 + RL::kK, p.K.codes + rowK * ROW, nt * kTile * ROW, bar);
          bulk_g2s(sb32 + RL::kV, p.V.codes + rowV * ROW, nt * kTile * ROW, bar);
          bulk_g2s(sb32 + RL::kRsK, reinterpret_cast<const unsigned char*>(p.K.rs) + rowK * 2, nt * kTile * 2, bar);
          bulk_g2s(sb32 + RL::kRsV, reinterpret_cast<const unsigned char*>(p.V.rs) + rowV * 2, nt * kTile * 2, bar);
          if constexpr (OUTL) {
            if (flk) bulk_g2s(sb32 + RL::kFlK, p.K.flags + rowK, nt * kTile * 4, bar);
            if (flv) bulk_g2s(sb32 + RL::kFlV, p.V.flags + rowV, nt * kTile * 4, bar);
            if (nK) bulk_g2s(sb32 + RL::kSideK, reinterpret_cast<const unsigned char*>(p.K.out_vals) + (bh * p.K.out_cap + ak) * 8, nK * 8, bar);
            if (nV) bulk_g2s(sb32 + RL::kPayV, reinterpret_cast<const unsigned char*>(p.V.out_vals) + (bh * p.V.out_cap + av) * 8, nV * 8, bar);
            if (nR) bulk_g2s(sb32 + RL::kSideK, p.K.ofrag + (bh * p.K.ofrag_cap + f0) * HQMQ_OFRAG_BYTES, nR * HQMQ_OFRAG_BYTES, bar);
          }
        }
        cur = nxt; kOff = kOffN; vOff = vOffN; fOff = fOffN;
      }
    }
    if (!ok) {
      if (lane == 0) { *abort_word = 1u; *p.status = p.epoch; }
    }
    // no copy may be in flight when the CTA exits: wait (bounded) for the stages that were issued last
    {
      const uint32_t n_back = gs < (uint32_t)NS ? gs : (uint32_t)NS;
      for (uint32_t k = 1; k <= n_back; ++k) {
        const uint32_t g = gs - k;
        uint32_t spins = 0;
        while (!mbar_try_wait(bar_full + 8 * (g % NS), (g / NS) & 1u) && ++spins < kWaitLimit) {}
      }
    }
    return;
  }

  // =============================== consumer warps =============================================================
  const int j = lane & 3, r = lane >> 2;
  // The V rows of a tile are read by four groups of lanes (j), each its tokens 2j and 2j + 1: with rows of 64 bytes
  // the four groups' loads would meet in the same banks (rows 0, 2, 4, 6 lie 128 bytes apart), so the odd groups
  // take their pair in the other order, and P is swapped to match (measured 280 -> 272 us per step on 64-byte rows;
  // on 32-byte rows the same trick measured no gain, other row sizes spread by themselves).
  constexpr int kVSwz = ROW % 128 == 64 ? 1 : 0;
  const int vswz = kVSwz == 1 ? (j & 1) : kVSwz == 2 ? ((j >> 1) & 1) : 0;
  const uint32_t pair_sel = vswz ? 0x1032u : 0x3210u;
  const uint32_t strideK = 8u << p.rep_log2, strideV = 8u << p.repv_log2;
  const uint32_t laneoffK = (uint32_t)(lane & ((1 << p.rep_log2) - 1)) * 8u;
  const uint32_t laneoffV = (uint32_t)(lane & ((1 << p.repv_log2) - 1)) * 8u;
  const int rows_f = p.table_rows >> 1;
  uint32_t gs = 0;
  bool failed = false;
  int cur_h = -1;
  FL ld;
  ld.row_bytes = ROW; ld.row_words = ROW / 4; ld.j = j; ld.r = r; ld.sdt = SDT;

  for (int u = u_first; (int64_t)u * p.tpu_v < flat_hi; ++u) {
    const UnitPiece up = unit_piece<N == 16>(p, u, flat_lo, flat_hi);
    const int h = up.h, b = up.b, tq = up.tq, t_beg = up.t_beg, t_end = up.t_end;
    // ---- tables of the KV head (sign-folded, replicated) and the unit's queries --------------------------------
    // (every consumer is past the previous unit's merge barrier here, so nobody still reads the old contents)
    if (h != cur_h) {
      const int repsK = 1 << p.rep_log2, repsV = 1 << p.repv_log2;
      const uint2* srcK = reinterpret_cast<const uint2*>(p.tblK) + (int64_t)h * p.table_rows;
      const uint2* srcV = reinterpret_cast<const uint2*>(p.tblV) + (int64_t)h * p.table_rows;
      // A warp loads 32 consecutive entries (one per lane) and writes their replicas -- entry after entry, `reps` copies
      // each, which is one contiguous stretch -- with lane-contiguous stores, the values passed by shuffles.  (One lane
      // storing all replicas of its own entry put every store of a warp into two banks: 4 us per table load.)
      for (int i0 = warp * 32; i0 < rows_f; i0 += kRingConsumerThreads) {
        const int i = i0 + lane;
        uint2 ek = make_uint2(0u, 0u), ev = make_uint2(0u, 0u);
        if (i < rows_f) { ek = srcK[2 * i]; ev = srcV[2 * i]; }
        uint2* dk = reinterpret_cast<uint2*>(tblK) + ((size_t)i0 << p.rep_log2);
        uint2* dv = reinterpret_cast<uint2*>(tblV) + ((size_t)i0 << p.repv_log2);
        for (int k = 0; k < repsK; ++k) {
          const int s = k * 32 + lane, from = s >> p.rep_log2;
          const uint2 v = make_uint2(__shfl_sync(0xffffffffu, ek.x, from), __shfl_sync(0xffffffffu, ek.y, from));
          if (i0 + from < rows_f) dk[s] = v;
        }
        for (int k = 0; k < repsV; ++k) {
          const int s = k * 32 + lane, from = s >> p.repv_log2;
          const uint2 v = make_uint2(__shfl_sync(0xffffffffu, ev.x, from), __shfl_sync(0xffffffffu, ev.y, from));
          if (i0 + from < rows_f) dv[s] = v;
        }
      }
      cur_h = h;
    }
    if constexpr (OUTL) {
      for (int i = threadIdx.x; i < 8 * D; i += kRingConsumerThreads) {
        const int g = i / D, x = i - g * D;
        qh16[g * qstride + x] = __float2half_rn(g < p.G ? load_float(p.Q, (int64_t)b * p.qs_b + (int64_t)tq * p.qs_t +
                                                                           (int64_t)(h * p.G + g) * p.qs_h + x, p.q_dtype) : 0.f);
      }
    }
    consumer_bar();

    // ---- Q as B fragments -------------------------------------------------------------------------------------
    uint32_t qb[NKS][2];
    {
      const int64_t q0off = (int64_t)b * p.qs_b + (int64_t)tq * p.qs_t;
#pragma unroll
      for (int ks = 0; ks < NKS; ++ks) {
        const int dim = 4 * (j * NKS + ks);
        float q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
        if (r < p.G) {
          const int64_t o = q0off + (int64_t)(h * p.G + r) * p.qs_h + dim;
          q0 = load_float(p.Q, o, p.q_dtype); q1 = load_float(p.Q, o + 1, p.q_dtype);
          q2 = load_float(p.Q, o + 2, p.q_dtype); q3 = load_float(p.Q, o + 3, p.q_dtype);
        }
        qb[ks][0] = pack_half2(q0, q1);
        qb[ks][1] = pack_half2(q2, q3);
      }
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NOT][4];
#pragma unroll
    for (int i = 0; i < NOT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const int64_t bh = (int64_t)b * p.Hkv + h;

    for (int tile0 = up.my_lo; tile0 < up.my_hi && !failed; tile0 += kRingTiles, ++gs) {
      const int buf = gs % NS;
      const int tile = tile0 + warp;
      // Every warp waits for the stage, also one without a tile in it (the last, partial stage of a piece): its
      // arrival on the "empty" barrier below must fall into THIS stage's phase, and only a completed "full" phase
      // proves that the producer has seen the previous use of the buffer released by all warps.
      if (!ring_wait(bar_full + 8 * buf, (gs / NS) & 1u, abort_word)) failed = true;
      failed = __any_sync(0xffffffffu, failed);
      if (failed) {
        if (lane == 0) { *abort_word = 1u; *p.status = p.epoch; }
        break;
      }
      if (tile < up.my_hi) {
        const unsigned char* sb = ring + (size_t)buf * RL::BYTES;
        const int t0 = tile * kTile;
        const bool edge = t0 < t_beg || t0 + kTile > t_end;
        const unsigned char* kc = sb + RL::kK + warp * (kTile * ROW);
        const unsigned char* vc = sb + RL::kV + warp * (kTile * ROW);

        // The tile, compiled twice: EDGE = false for a tile that lies wholly inside the key range (no masks, no
        // bounds on the rows), EDGE = true for the first / last tile of a range.
        auto tile_body = [&](auto edge_c) {
        constexpr bool EDGE = decltype(edge_c)::value;
        // ---- this lane's fields and scales ------------------------------------------------------------------
        typename FL::Raw cur;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int tr = nt * 8 + r;
          ld.template load_span<FL::KW, FL::LK>(cur.kw[nt], kc + tr * ROW, j, !EDGE || t0 + tr < t_end);
          cur.rsk[nt] = reinterpret_cast<const uint16_t*>(sb + RL::kRsK)[warp * kTile + tr];
          cur.rsv[nt] = reinterpret_cast<const uint16_t*>(sb + RL::kRsV)[warp * kTile + tr];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tr = 2 * j + ((i & 1) ^ vswz) + (i >> 1) * 8;
          ld.template load_span<FL::VW, FL::LV>(cur.vw[i], vc + tr * ROW, r, !EDGE || t0 + tr < t_end);
        }
        float ksc[2], vsc[2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          ksc[nt] = ld.kscale(cur, nt) * p.sscale;
          vsc[nt] = ld.vscale(cur, nt) * p.vscale;
        }
        bool okt[2] = {true, true};
        if constexpr (EDGE) {
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            const int t = t0 + nt * 8 + r;
            okt[nt] = t >= t_beg && t < t_end;
            if (!okt[nt]) vsc[nt] = 0.f;
          }
        }

        // ---- S^T = K Q^T -------------------------------------------------------------------------------------
        float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
        static_for<0, NKS>([&](auto ks_) {
          constexpr int ks = decltype(ks_)::value;
          uint32_t a[4];
          static_for<0, 2>([&](auto nt_) {
            constexpr int nt = decltype(nt_)::value;
            uint32_t idx; __half2 rr;
            FL::template cut<ks>(cur.kw[nt], idx, rr);
            const uint2 cw = *reinterpret_cast<const uint2*>(tblK + (idx * strideK + laneoffK));
            a[nt] = hmul2_u32(cw.x, rr);
            a[2 + nt] = hmul2_u32(cw.y, rr);
          });
          mma16816((ks & 1) ? s2 : s, a[0], a[1], a[2], a[3], qb[ks][0], qb[ks][1]);
        });

        // ---- K outliers ----------------------------------------------------------------------------------------
        float corr[4] = {0.f, 0.f, 0.f, 0.f};   // additions to the scaled scores (this lane's tokens r, r+8 x heads 2j, 2j+1)
        uint4 th0 = make_uint4(0u, 0u, 0u, 0u), sh0 = make_uint4(0u, 0u, 0u, 0u);
        if constexpr (OUTL) {
          th0 = *reinterpret_cast<const uint4*>(sb + RL::kTileHdr + warp * 32);                  // k0, k1, v0, v1
          const uint2 fr = *reinterpret_cast<const uint2*>(sb + RL::kTileHdr + warp * 32 + 16);   // f0, f1
          sh0 = *reinterpret_cast<const uint4*>(sb + RL::kStageHdr);                               // ak, nK, av, nV
          const uint2 sh1 = *reinterpret_cast<const uint2*>(sb + RL::kStageHdr + 16);             // first staged record, count
          if (fr.y > fr.x) {
            // fragment records: one 16-byte load per lane and one MMA per record (values and query in fp16,
            // the precision of the codeword path)
            uint32_t n = fr.y - fr.x; if (n > HQMQ_OFRAG_MAX_PER_TILE) n = HQMQ_OFRAG_MAX_PER_TILE;
            for (uint32_t g = 0; g < n; ++g) {
              const uint32_t ri = fr.x + g - sh1.x;        // index among the staged records
              uint32_t hdr;
              uint4 a;
              // (two loads per address space instead of one through a selected pointer: a generic load is served
              //  like a global one, and the staged record is the common case)
              if (ri < sh1.y) {
                const unsigned char* rec = sb + RL::kSideK + ri * HQMQ_OFRAG_BYTES;
                hdr = *reinterpret_cast<const uint32_t*>(rec);
                a = *reinterpret_cast<const uint4*>(rec + 16 + lane * 16);
              } else {
                const unsigned char* rec = p.K.ofrag + (bh * p.K.ofrag_cap + fr.x + g) * HQMQ_OFRAG_BYTES;
                hdr = __ldg(reinterpret_cast<const uint32_t*>(rec));
                a = __ldg(reinterpret_cast<const uint4*>(rec + 16 + lane * 16));
              }
              const uint32_t cj = (hdr >> (8 * j)) & 0xffu;
              uint2 qv = make_uint2(0u, 0u);
              if (cj != 0xffu) qv = *reinterpret_cast<const uint2*>(qh16 + r * qstride + 4 * cj);
              mma16816(s2, a.x, a.y, a.z, a.w, qv.x, qv.y);
            }
          } else if (th0.y > th0.x) {
            // no records: every flagged chunk adds <q_g, x> to the score of its token, one warp-wide step per chunk
            // (lane = head g * 4 + element; the products are summed over the element by two shuffles)
            uint32_t fw = 0;
            if (lane < kTile && t0 + lane < t_end) fw = reinterpret_cast<const uint32_t*>(sb + RL::kFlK)[warp * kTile + lane];
            uint32_t tm = __ballot_sync(0xffffffffu, fw != 0u);
            uint32_t e = th0.x;
            const int gq = lane >> 2, el = lane & 3;
            while (tm) {
              const int t = __ffs(tm) - 1;
              tm &= tm - 1;
              uint32_t w = __shfl_sync(0xffffffffu, fw, t);
              while (w) {
                const int c = __ffs(w) - 1;
                w &= w - 1;
                float xv = 0.f;
                if (e < (uint32_t)p.K.out_cap) {
                  const uint32_t rel = e - sh0.x;
                  if (p.K.out_dtype == HQMQ_F32) {
                    xv = reinterpret_cast<const float*>(p.K.out_vals)[(bh * p.K.out_cap + e) * 4 + el];
                  } else {
                    const uint16_t bits = rel < sh0.y ? reinterpret_cast<const uint16_t*>(sb + RL::kSideK)[rel * 4 + el]
                                                      : reinterpret_cast<const uint16_t*>(p.K.out_vals)[(bh * p.K.out_cap + e) * 4 + el];
                    xv = bits16_to_float(bits, p.K.out_dtype);
                  }
                }
                float pr = xv * __half2float(qh16[gq * qstride + 4 * c + el]);
                pr += __shfl_xor_sync(0xffffffffu, pr, 1);
                pr += __shfl_xor_sync(0xffffffffu, pr, 2);
                const float d0 = __shfl_sync(0xffffffffu, pr, 8 * j), d1 = __shfl_sync(0xffffffffu, pr, 8 * j + 4);
                if (r == (t & 7)) {
                  if (t & 8) { corr[2] += d0; corr[3] += d1; } else { corr[0] += d0; corr[1] += d1; }
                }
                ++e;
              }
            }
          }
        }
#pragma unroll
        for (int x = 0; x < 4; ++x) s[x] += s2[x];

        // ---- scale, mask, online softmax ---------------------------------------------------------------------
        // The reference exponent m_run of a head only has to bound the scores from above by a margin that keeps
        // 2^(s - m_run) and its sums in range; it is raised (and the accumulators rescaled) only when some score
        // of the tile exceeds it by more than kSlack, which after the first tiles of a range is rare.  The cross-lane
        // maximum (three shuffles per head) is taken only then.
        constexpr float kSlack = 4.f;
        float loc[2];
        bool need = false;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          s[e] = (!EDGE || okt[0]) ? fmaf(s[e], ksc[0], corr[e] * p.qscale) : -INFINITY;
          s[2 + e] = (!EDGE || okt[1]) ? fmaf(s[2 + e], ksc[1], corr[2 + e] * p.qscale) : -INFINITY;
          loc[e] = fmaxf(s[e], s[2 + e]);
          need |= loc[e] > m_run[e] + kSlack;
        }
        if (__any_sync(0xffffffffu, need)) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float m = loc[e];
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
            const float m_new = fmaxf(m_run[e], m);
            const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_run[e] - m_new);
            m_run[e] = m_new;
            l_run[e] *= alpha;
#pragma unroll
            for (int i = 0; i < NOT; ++i) { o[i][e] *= alpha; o[i][2 + e] *= alpha; }
          }
        }
        // P goes to the tensor cores as fp16(p * rs_V / qmax).  The weights that are summed into l (and that weigh the
        // V outliers below) are those rounded products divided by the same scale again, so numerator and denominator
        // of the output use one and the same set of weights: the rounding of P cancels instead of adding 2^-11 of
        // relative error to an output that a single key dominates.
        float pe[4];
        uint32_t pb[2];
        {
          float praw[4];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float m_use = m_run[e] == -INFINITY ? 0.f : m_run[e];
            praw[e] = fast_exp2(s[e] - m_use);
            praw[2 + e] = fast_exp2(s[2 + e] - m_use);
          }
          const __half2 h0 = __floats2half2_rn(praw[0] * vsc[0], praw[1] * vsc[0]);
          const __half2 h1 = __floats2half2_rn(praw[2] * vsc[1], praw[3] * vsc[1]);
          const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
          // (a token whose scale is zero -- an all-zero V row under fp16 scales -- adds nothing to the numerator but
          //  keeps its weight in the denominator; a masked token has weight 0 already)
          if (vsc[0] > 0.f) { const float iv0 = rcp_fast(vsc[0]); pe[0] = f0.x * iv0; pe[1] = f0.y * iv0; }
          else { pe[0] = praw[0]; pe[1] = praw[1]; }
          if (vsc[1] > 0.f) { const float iv1 = rcp_fast(vsc[1]); pe[2] = f1.x * iv1; pe[3] = f1.y * iv1; }
          else { pe[2] = praw[2]; pe[3] = praw[3]; }
          l_run[0] += pe[0] + pe[2];
          l_run[1] += pe[1] + pe[3];
          pb[0] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&h0));
          pb[1] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&h1));
          if constexpr (kVSwz != 0) {   // tokens 2j and 2j + 1 trade places where the V rows were loaded in the other order
            pb[0] = __byte_perm(pb[0], 0u, pair_sel);
            pb[1] = __byte_perm(pb[1], 0u, pair_sel);
          }
        }

        // ---- O^T += V^T P^T -----------------------------------------------------------------------------------
        static_for<0, NVG>([&](auto g_) {
          constexpr int g = decltype(g_)::value;
          uint32_t lo[4], hi[4];
          static_for<0, 4>([&](auto i_) {
            constexpr int i = decltype(i_)::value;
            uint32_t idx; __half2 rr;
            FL::template cut<g>(cur.vw[i], idx, rr);
            const uint2 cw = *reinterpret_cast<const uint2*>(tblV + (idx * strideV + laneoffV));
            lo[i] = hmul2_u32(cw.x, rr);
            hi[i] = hmul2_u32(cw.y, rr);
          });
          const uint32_t a0 = __byte_perm(lo[0], lo[1], 0x5410), a1 = __byte_perm(lo[0], lo[1], 0x7632);
          const uint32_t a2 = __byte_perm(lo[2], lo[3], 0x5410), a3 = __byte_perm(lo[2], lo[3], 0x7632);
          const uint32_t c0 = __byte_perm(hi[0], hi[1], 0x5410), c1 = __byte_perm(hi[0], hi[1], 0x7632);
          const uint32_t c2 = __byte_perm(hi[2], hi[3], 0x5410), c3 = __byte_perm(hi[2], hi[3], 0x7632);
          mma16816(o[2 * g], a0, a1, a2, a3, pb[0], pb[1]);
          mma16816(o[2 * g + 1], c0, c1, c2, c3, pb[0], pb[1]);
        });

        // ---- V outliers: o[g][4c + e] += P[t][g] * x[e] for every flagged chunk (t, c), in fp32 ------------------
        if constexpr (OUTL) {
          if (th0.w > th0.z) {
            uint32_t fw = 0;
            if (lane < kTile && t0 + lane < t_end) fw = reinterpret_cast<const uint32_t*>(sb + RL::kFlV)[warp * kTile + lane];
            // A tile whose flagged chunks sit in a few chunk columns (an outlier channel: one chunk of every token) takes
            // them column by column through the tensor cores: lane t < 16 turns token t's entry of the column into
            // fp16(x * qmax / rs) -- what the codeword path would have decoded had the chunk not been flagged -- the four
            // lanes that own the column's rows of V^T collect their tokens' values by shuffles, and two MMAs with the
            // tile's P add the column to the output.  About 45 warp instructions per column, whatever it holds; the
            // per-chunk fp32 step below costs about 25 per flagged chunk and stays the path of scattered outliers.
            // (compiled for d_head 64 only, like its predecessor, a patch of the decoded fragments inside the V loop:
            //  in the d_head 128 kernels any addition to the tile costs registers that the common path needs)
            bool by_column = false;
            if constexpr (N == 16) {
              const uint32_t cnt = th0.w - th0.z;
              if (cnt > 5u) {
                const uint32_t cols = __reduce_or_sync(0xffffffffu, fw);
                float rsv = 1.f;
                if (lane < kTile) rsv = bits16_to_float(reinterpret_cast<const uint16_t*>(sb + RL::kRsV)[warp * kTile + lane], SDT);
                // (P reaches the tensor cores multiplied by the token's scale, so a flagged chunk in a token whose
                //  stored scale is zero -- a scale below the range of its 16-bit type -- cannot be carried that way)
                const bool zero_scale = __any_sync(0xffffffffu, fw != 0u && !(rsv > 0.f));
                by_column = !zero_scale && (uint32_t)__popc(cols) * 8u < cnt * 5u;
                if (by_column) {
                  const float inv = __fdividef(p.qmaxf, rsv);
                  const uint32_t ex = excl_scan16(__popc(fw), lane);
                  uint32_t left = cols;
                  while (left) {
                    const int c = __ffs(left) - 1;
                    left &= left - 1;
                    uint32_t xlo = 0u, xhi = 0u;
                    if ((fw >> c) & 1u) {
                      const uint32_t e = th0.z + ex + __popc(fw & ((1u << c) - 1u));
                      if (e < (uint32_t)p.V.out_cap) {
                        float x0, x1, x2, x3;
                        if (p.V.out_dtype == HQMQ_F32) {
                          const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.V.out_vals) + (bh * p.V.out_cap + e) * 4);
                          x0 = v.x; x1 = v.y; x2 = v.z; x3 = v.w;
                        } else {
                          const uint32_t rel = e - sh0.z;
                          uint2 v;
                          if (rel < sh0.w) v = reinterpret_cast<const uint2*>(sb + RL::kPayV)[rel];
                          else v = __ldg(reinterpret_cast<const uint2*>(p.V.out_vals) + bh * p.V.out_cap + e);
                          const float2 a = pair16_to_float2(v.x, p.V.out_dtype), bb = pair16_to_float2(v.y, p.V.out_dtype);
                          x0 = a.x; x1 = a.y; x2 = bb.x; x3 = bb.y;
                        }
                        xlo = pack_half2(x0 * inv, x1 * inv);
                        xhi = pack_half2(x2 * inv, x3 * inv);
                      }
                    }
                    // rows r and r + 8 of the MMA's A operand are elements 0 and 1 (then 2 and 3) of chunk r * NVG + g;
                    // the lanes of other rows fetch from lane 31, which holds zeros
                    const bool mine = r == c / NVG;
                    uint32_t lo[4], hi[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                      const int src = mine ? 2 * j + ((i & 1) ^ vswz) + (i >> 1) * 8 : 31;
                      lo[i] = __shfl_sync(0xffffffffu, xlo, src);
                      hi[i] = __shfl_sync(0xffffffffu, xhi, src);
                    }
                    const uint32_t a0 = __byte_perm(lo[0], lo[1], 0x5410), a1 = __byte_perm(lo[0], lo[1], 0x7632);
                    const uint32_t a2 = __byte_perm(lo[2], lo[3], 0x5410), a3 = __byte_perm(lo[2], lo[3], 0x7632);
                    const uint32_t c0 = __byte_perm(hi[0], hi[1], 0x5410), c1 = __byte_perm(hi[0], hi[1], 0x7632);
                    const uint32_t c2 = __byte_perm(hi[2], hi[3], 0x5410), c3 = __byte_perm(hi[2], hi[3], 0x7632);
                    static_for<0, NVG>([&](auto gg_) {
                      constexpr int gg = decltype(gg_)::value;
                      if (c % NVG == gg) {
                        mma16816(o[2 * gg], a0, a1, a2, a3, pb[0], pb[1]);
                        mma16816(o[2 * gg + 1], c0, c1, c2, c3, pb[0], pb[1]);
                      }
                    });
                  }
                }
              }
            }
            if (!by_column) {
            uint32_t tm = __ballot_sync(0xffffffffu, fw != 0u);
            uint32_t e = th0.z;
            while (tm) {
              const int t = __ffs(tm) - 1;
              tm &= tm - 1;
              uint32_t w = __shfl_sync(0xffffffffu, fw, t);
              // P of token t for heads 2j, 2j+1 lives in the lane with r = t & 7 and the same j
              const int src = ((t & 7) << 2) | j;
              const float p0 = __shfl_sync(0xffffffffu, (t & 8) ? pe[2] : pe[0], src);
              const float p1 = __shfl_sync(0xffffffffu, (t & 8) ? pe[3] : pe[1], src);
              while (w) {
                const int c = __ffs(w) - 1;
                w &= w - 1;
                float x0 = 0.f, x1 = 0.f, x2 = 0.f, x3 = 0.f;
                if (e < (uint32_t)p.V.out_cap) {
                  if (p.V.out_dtype == HQMQ_F32) {
                    const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.V.out_vals) + (bh * p.V.out_cap + e) * 4);
                    x0 = v.x; x1 = v.y; x2 = v.z; x3 = v.w;
                  } else {
                    const uint32_t rel = e - sh0.z;
                    const uint2 v = rel < sh0.w ? reinterpret_cast<const uint2*>(sb + RL::kPayV)[rel]
                                                : reinterpret_cast<const uint2*>(p.V.out_vals)[bh * p.V.out_cap + e];
                    const float2 a = pair16_to_float2(v.x, p.V.out_dtype), bb = pair16_to_float2(v.y, p.V.out_dtype);
                    x0 = a.x; x1 = a.y; x2 = bb.x; x3 = bb.y;
                  }
                }
                if (r == c / NVG) {
                  static_for<0, NVG>([&](auto gg_) {
                    constexpr int gg = decltype(gg_)::value;
                    if (c % NVG == gg) {
                      o[2 * gg][0] = fmaf(p0, x0, o[2 * gg][0]); o[2 * gg][1] = fmaf(p1, x0, o[2 * gg][1]);
                      o[2 * gg][2] = fmaf(p0, x1, o[2 * gg][2]); o[2 * gg][3] = fmaf(p1, x1, o[2 * gg][3]);
                      o[2 * gg + 1][0] = fmaf(p0, x2, o[2 * gg + 1][0]); o[2 * gg + 1][1] = fmaf(p1, x2, o[2 * gg + 1][1]);
                      o[2 * gg + 1][2] = fmaf(p0, x3, o[2 * gg + 1][2]); o[2 * gg + 1][3] = fmaf(p1, x3, o[2 * gg + 1][3]);
                    }
                  });
                }
                ++e;
              }
            }
            }   // !by_column
          }
        }
        };   // tile_body
        if (edge) tile_body(std::true_type{});
        else tile_body(std::false_type{});
        __syncwarp();   // every lane is done with the stage before lane 0 releases it
      }
      if (lane == 0) mbar_arrive(bar_empty + 8 * buf);
    }

    // ---- one partial per (CTA, unit, head): the warps' results are merged in shared memory, in a fixed order ----
    if (consumer_bar_or(failed)) break;
    {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float l = l_run[e];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        if (r == 0) { m_s[warp * 8 + 2 * j + e] = m_run[e]; l_s[warp * 8 + 2 * j + e] = l; }
      }
    }
    consumer_bar();
    if (threadIdx.x < kRingWarps * 8) {
      const int w = threadIdx.x >> 3, g = threadIdx.x & 7;
      float m_star = -INFINITY;
#pragma unroll
      for (int i = 0; i < kRingWarps; ++i) m_star = fmaxf(m_star, m_s[i * 8 + g]);
      const float m_use = m_star == -INFINITY ? 0.f : m_star;
      w_s[w * 8 + g] = fast_exp2(m_s[w * 8 + g] - m_use);     // 0 for a warp that saw no key
      if (w == 0) {
        float l_star = 0.f;
#pragma unroll
        for (int i = 0; i < kRingWarps; ++i) l_star = fmaf(l_s[i * 8 + g], fast_exp2(m_s[i * 8 + g] - m_use), l_star);
        ms_s[g] = m_star; ms_s[8 + g] = l_star;
      }
    }
    consumer_bar();
    {
      const int MS = p.merge_slots;
      constexpr int PER = (8 * D + kRingConsumerThreads - 1) / kRingConsumerThreads;   // elements of [8][D] per thread
      float acc[PER];
#pragma unroll
      for (int q = 0; q < PER; ++q) acc[q] = 0.f;
      const float wg0 = w_s[warp * 8 + 2 * j], wg1 = w_s[warp * 8 + 2 * j + 1];
      // Where element x of head pair jj sits in a slot row.  The lanes of a store differ in r (bits 6:4 of x at d_head
      // 128, 5:3 at 64) and in j, which as plain indices would all fall into two banks (16-way conflicts, 4 us per
      // merge): the upper bits of r are folded into bits 3:2 and j into bits 1:0, which spreads a store over all 32
      // banks.  The map is its own inverse (it changes bits 3:0 only, by bits it leaves alone).
      auto slot_swz = [](int jj, int x) { return x ^ (((x >> 5) & (D / 32 - 1)) << 2) ^ (jj & 3); };
      // (15 warps: the host picks a divisor of 15 as slot count; otherwise the last round fills only some of the slots)
      constexpr bool kWhole = kRingWarps % 15 == 0;
      const int rounds = kWhole ? kRingWarps / MS : (kRingWarps + MS - 1) / MS;
      for (int round = 0; round < rounds; ++round) {
        const int live = kWhole ? MS : min(MS, kRingWarps - round * MS);
        if (warp / MS == round) {
          float* mine = slots + (size_t)(warp % MS) * 8 * D;
#pragma unroll
          for (int i = 0; i < NOT; ++i) {
            const int chunk = r * NVG + (i >> 1);
            if (chunk < N) {
              const int x = 4 * chunk + 2 * (i & 1);
              mine[(2 * j) * D + slot_swz(j, x)] = o[i][0] * wg0;              // row r (element 0 / 2), head 2j
              mine[(2 * j + 1) * D + slot_swz(j, x)] = o[i][1] * wg1;          // head 2j+1
              mine[(2 * j) * D + slot_swz(j, x + 1)] = o[i][2] * wg0;          // row r+8 (element 1 / 3)
              mine[(2 * j + 1) * D + slot_swz(j, x + 1)] = o[i][3] * wg1;
            }
          }
        }
        consumer_bar();
#pragma unroll
        for (int q = 0; q < PER; ++q) {
          const int i = threadIdx.x + q * kRingConsumerThreads;
          if (i < 8 * D)
            for (int sidx = 0; sidx < live; ++sidx) acc[q] += slots[(size_t)sidx * 8 * D + i];
        }
        consumer_bar();
      }
      // ---- across the CTAs that share the unit: the last one to finish merges all of their partials ----------------
      // (no CTA waits for another: a ticket per unit counts arrivals, and whoever draws the last one does the merge)
      const int64_t ubase = (int64_t)u * p.tpu_v;
      const int c0 = (int)(ubase / p.L), n_ctas = (int)((ubase + p.tpu_v - 1) / p.L) - c0 + 1;
      auto emit = [&](int g, int x, float v, float m_star, float l_star) {
        const int64_t row = ((int64_t)b * p.Hq + h * p.G + g) * p.Tq + tq;
        if (p.merged) {
          p.merged[row * (D + 2) + x] = v;
          if (x == 0) { p.merged[row * (D + 2) + D] = m_star; p.merged[row * (D + 2) + D + 1] = l_star; }
        } else {
          store_float(p.O, (int64_t)b * p.os_b + (int64_t)(h * p.G + g) * p.os_h + (int64_t)tq * p.os_t + x,
                      l_star > 0.f ? v / l_star : 0.f, p.o_dtype);
        }
      };
      if (n_ctas == 1) {
#pragma unroll
        for (int q = 0; q < PER; ++q) {
          const int i = threadIdx.x + q * kRingConsumerThreads;
          if (i < 8 * D) {
            const int g = i / D, x = slot_swz(g >> 1, i - g * D);
            if (g < p.G) emit(g, x, acc[q], ms_s[g], ms_s[8 + g]);
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < PER; ++q) {
          const int i = threadIdx.x + q * kRingConsumerThreads;
          if (i < 8 * D) {
            const int g = i / D, x = slot_swz(g >> 1, i - g * D);
            if (g < p.G) {
              const int64_t row = ((int64_t)b * p.Hq + h * p.G + g) * p.Tq + tq;
              float* dst = p.partials + (row * p.P + up.part) * (D + 2);
              dst[x] = acc[q];
              if (x == 0) { dst[D] = ms_s[g]; dst[D + 1] = ms_s[8 + g]; }
            }
          }
        }
        __threadfence();                      // this CTA's partial is visible device-wide before its ticket is drawn
        consumer_bar();
        if (threadIdx.x == 0) *last_s = atomicAdd(&p.tickets[u], 1u) == (uint32_t)(n_ctas - 1) ? 1u : 0u;
        consumer_bar();
        if (*last_s) {
          __threadfence();
#pragma unroll
          for (int q = 0; q < PER; ++q) {
            const int i = threadIdx.x + q * kRingConsumerThreads;
            if (i < 8 * D) {
              const int g = i / D, x = i - g * D;
              if (g < p.G) {
                const int64_t row = ((int64_t)b * p.Hq + h * p.G + g) * p.Tq + tq;
                const float* base = p.partials + row * p.P * (D + 2);
                float m_star = -INFINITY;
                for (int c = 0; c < n_ctas; ++c) m_star = fmaxf(m_star, __ldcg(base + c * (D + 2) + D));
                const float m_use = m_star == -INFINITY ? 0.f : m_star;
                float v = 0.f, l_star = 0.f;
                for (int c = 0; c < n_ctas; ++c) {
                  const float wgt = fast_exp2(__ldcg(base + c * (D + 2) + D) - m_use);
                  v = fmaf(__ldcg(base + c * (D + 2) + x), wgt, v);
                  l_star = fmaf(__ldcg(base + c * (D + 2) + D + 1), wgt, l_star);
                }
                emit(g, x, v, m_star, l_star);
              }
            }
          }
        }
      }
    }
    // (the next unit's table / query writes and the next merge are ordered behind this unit's reads by the
    //  barrier at the top of the next unit and by the merge barriers themselves)
    consumer_bar();
  }
}

}  // namespace attn
}  // namespace hqmq
