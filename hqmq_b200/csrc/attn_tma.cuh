// Decode attention over the native compressed cache with the KV tiles staged through shared memory
// by bulk asynchronous copies (cp.async.bulk + mbarrier), one CTA per SM.
//
// Every warp owns a ring of kStages tile buffers.  One lane issues, for the tile kStages-1 ahead, one
// bulk copy per plane piece (16 code rows of K, 16 of V, the two scale vectors, and with Med3x the flag
// words and the tile's slice of the outlier side buffers); all lanes wait on the stage's mbarrier and
// then cut their bit fields out of shared memory.  Compared with prefetching into registers this keeps
// several tiles in flight per warp at a cost of no registers, so more warps fit on the SM.
// The arithmetic (fragment layouts, softmax, outlier handling) is the one described in attn_kernel.cuh.
#pragma once
#include "attn_kernel.cuh"

namespace hqmq {
namespace attn {

constexpr int kStages = 2;
constexpr int kPay = 64;                 // outlier entries staged per tile and tensor (+2 alignment slack)
constexpr uint32_t kWaitLimit = 1u << 24;
// bytes of a stage that hold either the K payload slice or the tile's fragment records
constexpr int kSideK = (kPay + 2) * 8 > HQMQ_OFRAG_MAX_PER_TILE * HQMQ_OFRAG_BYTES ? (kPay + 2) * 8
                                                                                  : HQMQ_OFRAG_MAX_PER_TILE * HQMQ_OFRAG_BYTES;
constexpr int kQPad = 8;   // halves of padding per query row in shared memory (spreads the rows over banks)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

// Shared-memory layout of one stage (all pieces 16-byte aligned).
template <int N, int IB, int RB, bool OUTL>
struct StageLayout {
  static constexpr int ROW = N * (IB + RB) / 8;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTile * ROW;
  static constexpr int kRsK = kV + kTile * ROW;
  static constexpr int kRsV = kRsK + 32;
  static constexpr int kFlK = kRsV + 32;
  static constexpr int kFlV = kFlK + 64;
  static constexpr int kPayK = kFlV + 64;               // K side-buffer slice, or the tile's fragment records
  static constexpr int kPayV = kPayK + kSideK;
  static constexpr int kHdr = kPayV + (kPay + 2) * 8;   // off0K, off0V, fragment records, staged-flags bits
  static constexpr int BYTES = OUTL ? kHdr + 16 : kFlK;
  static_assert((kTile * ROW) % 16 == 0, "tile of code rows must be a multiple of 16 bytes");
};

template <int N, int IB, int RB, int NW, bool OUTL>
__device__ __forceinline__ void attn_decode_tma_body(const AttnParams& p, uint32_t* status) {
  using G_ = Geo<N>;
  constexpr bool FOLD = !OUTL;   // the outlier kernel is issue-bound: it keeps the full table and the shorter gather
  using FL = FastLoader<N, IB, RB, FOLD>;
  using SL = StageLayout<N, IB, RB, OUTL>;
  constexpr int NKS = G_::NKS, NVG = G_::NVG, NOT = 2 * G_::NVG;
  constexpr int NHEADS = 8;
  constexpr int ROW = SL::ROW;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t rstride = 8u << p.rep_log2;
  const int rows_f = FOLD ? p.table_rows >> 1 : p.table_rows;   // sign-folded tables keep the even native indices only
  const size_t tbl_bytes = (size_t)rows_f * rstride;
  unsigned char* tblK = smem_raw;
  unsigned char* tblV = smem_raw + tbl_bytes;
  // Warp mode (p.warp_units): the warps of a CTA work on different units at the same time -- see the unit loop.
  const bool wm = p.warp_units != 0;
  const int qstride = p.d + kQPad;
  // [8][d] queries of the unit in fp16 (OUTL); in warp mode every warp has its own copy
  __half* qh16 = reinterpret_cast<__half*>(smem_raw + 2 * tbl_bytes) + (wm ? (size_t)(threadIdx.x >> 5) * NHEADS * qstride : 0);
  unsigned char* after_q = smem_raw + 2 * tbl_bytes + (OUTL ? (size_t)(wm ? NW : 1) * NHEADS * qstride * 2 : 0);
  uint64_t* bars = reinterpret_cast<uint64_t*>(after_q);                                      // [NW][kStages]
  unsigned char* warp_area = after_q + ((NW * kStages * 8 + 15) & ~15);
  // per-warp share of the staging area; it also holds one warp's partial [8 heads][d + 2] during the merge
  constexpr int WARP_BYTES = kStages * SL::BYTES > NHEADS * (4 * N + 2) * 4 ? kStages * SL::BYTES : NHEADS * (4 * N + 2) * 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = lane & 3, r = lane >> 2;
  const uint32_t lane_off = (uint32_t)(lane & ((1 << p.rep_log2) - 1)) * 8u;
  unsigned char* my_area = warp_area + (size_t)warp * WARP_BYTES;
  const uint32_t bar0 = smem_u32(bars + warp * kStages);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) mbar_init(bar0 + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  uint32_t it = 0;        // tiles this warp has consumed so far (stage = it % kStages, parity from it / kStages)
  bool failed = false, drained = false;

  const int64_t flat_lo = (int64_t)blockIdx.x * p.L;
  const int64_t flat_total = (int64_t)p.units * p.tpu_v;
  const int64_t flat_hi = flat_lo + p.L < flat_total ? flat_lo + p.L : flat_total;
  const int upb = p.B * p.Tq;
  int cur_h = -1;

  for (int u = (int)(flat_lo / p.tpu_v); (int64_t)u * p.tpu_v < flat_hi; ++u) {
    const int h = u / upb, bt = u - h * upb;
    const int b = bt / p.Tq, tq = bt - b * p.Tq;
    // CTA mode: all warps share the unit -- barriers around the tables and the staged queries of every unit, the warps'
    // results merged in shared memory at its end.  Warp mode (units of a few tiles each, many of them per CTA): the
    // CTA's tiles go round-robin to its warps over the whole flat range, every warp runs through the units on its
    // own -- its queries staged in its own copy, its partial written to its own slot, empty where it had no tile --
    // and the CTA meets only where the KV head, and with it the tables, changes.  (In CTA mode a unit of ten tiles kept
    // six of sixteen warps idle and every unit paid barriers, a merge and the latency of its first copies in turn:
    // 42 us for 512 units of ten tiles at d_head 64.)
    if (wm ? h != cur_h : (h != cur_h || OUTL)) __syncthreads();
    if (h != cur_h) {
      const int reps = 1 << p.rep_log2;
      for (int i = threadIdx.x; i < rows_f; i += NW * 32) {
        const uint2 ek = (reinterpret_cast<const uint2*>(p.tblK) + (int64_t)h * p.table_rows)[FOLD ? 2 * i : i];
        const uint2 ev = (reinterpret_cast<const uint2*>(p.tblV) + (int64_t)h * p.table_rows)[FOLD ? 2 * i : i];
        uint2* dk = reinterpret_cast<uint2*>(tblK + (size_t)i * rstride);
        uint2* dv = reinterpret_cast<uint2*>(tblV + (size_t)i * rstride);
        for (int q = 0; q < reps; ++q) { dk[q] = ek; dv[q] = ev; }
      }
      cur_h = h;
      if (wm) __syncthreads();
    }
    if (!wm) {
      if constexpr (OUTL) {
        for (int i = threadIdx.x; i < NHEADS * p.d; i += NW * 32) {
          const int g = i / p.d, x = i - g * p.d;
          qh16[g * qstride + x] = __float2half_rn(g < p.G ? load_float(p.Q, (int64_t)b * p.qs_b + (int64_t)tq * p.qs_t +
                                                                             (int64_t)(h * p.G + g) * p.qs_h + x, p.q_dtype) : 0.f);
        }
      }
      __syncthreads();
    }

    int t_beg, t_end;
    key_range(p.Tkv, p.Tq, p.causal, p.window, tq, t_beg, t_end);
    const int tile_lo = t_beg / kTile, tile_hi = (t_end + kTile - 1) / kTile;
    const int64_t ubase = (int64_t)u * p.tpu_v;
    const int rel_lo = (int)(flat_lo > ubase ? flat_lo - ubase : 0);
    const int rel_hi = (int)(flat_hi < ubase + p.tpu_v ? flat_hi - ubase : p.tpu_v);
    const int my_lo = tile_lo + rel_lo;
    const int my_hi = min(tile_hi, tile_lo + rel_hi);
    const int part = (int)blockIdx.x - (int)(ubase / p.L);   // this CTA's slot among the CTAs that share the unit
    // this warp's first tile of the piece is my_lo + w0: the warp's own index, or in warp mode its turn in the
    // round-robin over the CTA's flat range
    int w0 = warp;
    if (wm) {
      const int lo_i = (int)(ubase + (my_lo - tile_lo) - flat_lo);
      w0 = (warp - lo_i % NW + NW) % NW;
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NOT][4];
#pragma unroll
    for (int i = 0; i < NOT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    // ---- producer side (lane 0): the bulk copies of one tile ----------------------------------------------
    // Plane addresses are rebuilt from the launch parameters at every use instead of being held in registers:
    // only one lane needs them, and twelve 64-bit pointers per thread would push the loop into spills.
    const int64_t bh = (int64_t)b * p.Hkv + h;
    const bool hasFlK = OUTL && p.K.flags != nullptr, hasFlV = OUTL && p.V.flags != nullptr;
    const bool stageK = hasFlK && p.K.out_dtype != HQMQ_F32, stageV = hasFlV && p.V.out_dtype != HQMQ_F32;
    const bool hasFr = hasFlK && p.K.ofrag != nullptr;
    uint32_t nk0 = 0, nk1 = 0, nv0 = 0, nv1 = 0, nf0 = 0, nf1 = 0;   // payload / record ranges of the tile to be issued next
    auto load_offsets = [&](int tl) {
      nk0 = nk1 = nv0 = nv1 = nf0 = nf1 = 0;
      if (tl < my_hi) {
        if (hasFlK) {
          const uint32_t* o = p.K.out_off + bh * (p.K.T_cap / HQMQ_OUT_BLOCK + 1) + tl;
          nk0 = o[0]; nk1 = o[1];
        }
        if (hasFlV) {
          const uint32_t* o = p.V.out_off + bh * (p.V.T_cap / HQMQ_OUT_BLOCK + 1) + tl;
          nv0 = o[0]; nv1 = o[1];
        }
        if (hasFr) {
          const uint32_t* o = p.K.ofrag_off + bh * (p.K.T_cap / HQMQ_OUT_BLOCK + 1) + tl;
          nf0 = o[0]; nf1 = o[1];
        }
      }
    };
    auto issue = [&](int tl, uint32_t seq) {   // lane 0 only
      const int st = seq % kStages;
      unsigned char* sb = my_area + st * SL::BYTES;
      const uint32_t sb32 = smem_u32(sb), bar = bar0 + 8 * st;
      uint32_t bytes = 2 * kTile * ROW + 64;
      uint32_t pk_bytes = 0, pv_bytes = 0, fr_bytes = 0, ak = 0, av = 0;
      bool flk = false, flv = false;   // does this tile need its flag words (it has side-buffer entries to merge)
      if constexpr (OUTL) {
        uint32_t nfr = 0;
        if (nf1 > nf0) {
          // the tile owns fragment records: they replace its K flag words and payload slice
          nfr = nf1 - nf0; if (nfr > HQMQ_OFRAG_MAX_PER_TILE) nfr = HQMQ_OFRAG_MAX_PER_TILE;
          fr_bytes = nfr * HQMQ_OFRAG_BYTES; bytes += fr_bytes;
        } else if (nk1 > nk0) {
          flk = true; bytes += 64;
          if (stageK) {
            // (entries at or beyond out_cap were dropped by the encoder: nothing of them is copied, they read as 0)
            ak = nk0 & ~1u;
            uint32_t n = nk1 - ak; if (n > kPay + 1) n = kPay + 1;
            const uint32_t room = ak < (uint32_t)p.K.out_cap ? (uint32_t)p.K.out_cap - ak : 0u;
            if (n > room) n = room;
            pk_bytes = ((n + 1) & ~1u) * 8; bytes += pk_bytes;
          }
        }
        if (nv1 > nv0) {
          flv = true; bytes += 64;
          if (stageV) {
            av = nv0 & ~1u;
            uint32_t n = nv1 - av; if (n > kPay + 1) n = kPay + 1;
            const uint32_t room = av < (uint32_t)p.V.out_cap ? (uint32_t)p.V.out_cap - av : 0u;
            if (n > room) n = room;
            pv_bytes = ((n + 1) & ~1u) * 8; bytes += pv_bytes;
          }
        }
        *reinterpret_cast<uint4*>(sb + SL::kHdr) = make_uint4(nk0, nv0, nfr, (flk ? 1u : 0u) | (flv ? 2u : 0u));
      }
      mbar_expect_tx(bar, bytes);
      const int64_t rowK = bh * p.K.T_cap + (int64_t)tl * kTile, rowV = bh * p.V.T_cap + (int64_t)tl * kTile;
      bulk_g2s(sb32 + SL::kK, p.K.codes + rowK * ROW, kTile * ROW, bar);
      bulk_g2s(sb32 + SL::kV, p.V.codes + rowV * ROW, kTile * ROW, bar);
      bulk_g2s(sb32 + SL::kRsK, reinterpret_cast<const unsigned char*>(p.K.rs) + rowK * 2, 32, bar);
      bulk_g2s(sb32 + SL::kRsV, reinterpret_cast<const unsigned char*>(p.V.rs) + rowV * 2, 32, bar);
      if constexpr (OUTL) {
        if (flk) bulk_g2s(sb32 + SL::kFlK, p.K.flags + rowK, 64, bar);
        if (flv) bulk_g2s(sb32 + SL::kFlV, p.V.flags + rowV, 64, bar);
        if (fr_bytes) bulk_g2s(sb32 + SL::kPayK, p.K.ofrag + (bh * p.K.ofrag_cap + nf0) * HQMQ_OFRAG_BYTES, fr_bytes, bar);
        if (pk_bytes)
          bulk_g2s(sb32 + SL::kPayK, reinterpret_cast<const unsigned char*>(p.K.out_vals) + (bh * p.K.out_cap + ak) * 8, pk_bytes, bar);
        if (pv_bytes)
          bulk_g2s(sb32 + SL::kPayV, reinterpret_cast<const unsigned char*>(p.V.out_vals) + (bh * p.V.out_cap + av) * 8, pv_bytes, bar);
      }
    };

    // (a warp that gave up on a wait takes no more tiles; in warp mode it still walks the units, for the barriers)
    const int n_my = !failed && my_hi > my_lo + w0 ? (my_hi - my_lo - w0 + NW - 1) / NW : 0;
    // prologue: kStages-1 tiles in flight
    if (lane == 0 && !failed) {
      if constexpr (OUTL) load_offsets(my_lo + w0);
#pragma unroll
      for (int k = 0; k < kStages - 1; ++k) {
        if (k < n_my) {
          issue(my_lo + w0 + k * NW, it + k);
          if constexpr (OUTL) load_offsets(my_lo + w0 + (k + 1) * NW);
        }
      }
    }

    // ---- Q as B fragments (loaded while the first copies are in flight) ------------------------------------------
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
    if constexpr (OUTL) {
      if (wm) {   // the lanes of a warp hold all 8 x d query values between them: park them for the outlier paths
#pragma unroll
        for (int ks = 0; ks < NKS; ++ks)
          *reinterpret_cast<uint2*>(qh16 + r * qstride + 4 * (j * NKS + ks)) = make_uint2(qb[ks][0], qb[ks][1]);
        __syncwarp();
      }
    }
    for (int k = 0; k < n_my && !failed; ++k, ++it) {
      const int tile = my_lo + w0 + k * NW;
      if (lane == 0 && k + kStages - 1 < n_my) {
        issue(tile + (kStages - 1) * NW, it + kStages - 1);
        if constexpr (OUTL) load_offsets(tile + kStages * NW);
      }
      const int st = it % kStages;
      const uint32_t parity = (it / kStages) & 1u;
      {
        uint32_t spins = 0;
        while (!mbar_try_wait(bar0 + 8 * st, parity)) {
          if (++spins > kWaitLimit) { failed = true; break; }
        }
        failed = __any_sync(0xffffffffu, failed);
        if (failed) { if (lane == 0) *status = p.epoch; break; }
        __syncwarp();
      }
      const unsigned char* sb = my_area + st * SL::BYTES;
      const int t0 = tile * kTile;
      const bool edge = t0 < t_beg || t0 + kTile > t_end;

      // ---- this lane's fields and scales out of the stage ------------------------------------------------
      typename FL::Raw cur;
      FL ld;
      ld.row_bytes = ROW; ld.row_words = ROW / 4; ld.j = j; ld.r = r; ld.sdt = p.K.scale_dtype;
      ld.set_table(rstride, lane_off);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int tr = nt * 8 + r;
        ld.template load_span<FL::KW, FL::LK>(cur.kw[nt], sb + SL::kK + tr * ROW, j, !edge || t0 + tr < t_end);
        cur.rsk[nt] = reinterpret_cast<const uint16_t*>(sb + SL::kRsK)[tr];
        cur.rsv[nt] = reinterpret_cast<const uint16_t*>(sb + SL::kRsV)[tr];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tr = 2 * j + (i & 1) + (i >> 1) * 8;
        ld.template load_span<FL::VW, FL::LV>(cur.vw[i], sb + SL::kV + tr * ROW, r, !edge || t0 + tr < t_end);
      }
      float ksc[2], vsc[2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        ksc[nt] = ld.kscale(cur, nt) * p.sscale;
        vsc[nt] = ld.vscale(cur, nt) * p.vscale;
      }
      bool okt[2] = {true, true};
      if (edge) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int t = t0 + nt * 8 + r;
          okt[nt] = t >= t_beg && t < t_end;
          if (!okt[nt]) vsc[nt] = 0.f;
        }
      }

      // ---- outliers --------------------------------------------------------------------------------------
      bool anyK = false, anyV = false;
      uint32_t offk = 0, offv = 0, fv_tile = 0, fk_tile = 0, nfr = 0;
      if constexpr (OUTL) {
        const uint4 hdr = *reinterpret_cast<const uint4*>(sb + SL::kHdr);
        offk = hdr.x; offv = hdr.y; nfr = hdr.z;
        uint32_t fk = 0, fv = 0;
        if (hdr.w && lane < 16 && t0 + lane < t_end) {
          if (hdr.w & 1u) fk = reinterpret_cast<const uint32_t*>(sb + SL::kFlK)[lane];
          if (hdr.w & 2u) fv = reinterpret_cast<const uint32_t*>(sb + SL::kFlV)[lane];
        }
        (void)hasFlK; (void)hasFlV;
        anyK = (hdr.w & 1u) && __ballot_sync(0xffffffffu, fk != 0) != 0;
        anyV = (hdr.w & 2u) && __ballot_sync(0xffffffffu, fv != 0) != 0;
        fv_tile = fv; fk_tile = fk;
      }

      // ---- S^T = K Q^T ----------------------------------------------------------------------------------------
      float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
      static_for<0, NKS>([&](auto ks_) {
        constexpr int ks = decltype(ks_)::value;
        uint32_t a[4];
        static_for<0, 2>([&](auto nt_) {
          constexpr int nt = decltype(nt_)::value;
          uint32_t idx; __half2 rr;
          ld.template koff<nt, ks>(cur, idx, rr);
          const uint2 cw = *reinterpret_cast<const uint2*>(tblK + idx);
          a[nt] = hmul2_u32(cw.x, rr);
          a[2 + nt] = hmul2_u32(cw.y, rr);
        });
        mma16816((ks & 1) ? s2 : s, a[0], a[1], a[2], a[3], qb[ks][0], qb[ks][1]);
      });
      if constexpr (OUTL) {
        // K outliers of a tile that owns fragment records: one shared-memory load and one MMA per record (values
        // and query in fp16, the precision the codeword path has too)
        for (uint32_t g = 0; g < nfr; ++g) {
          const unsigned char* rec = sb + SL::kPayK + g * HQMQ_OFRAG_BYTES;
          const uint32_t cj = (*reinterpret_cast<const uint32_t*>(rec) >> (8 * j)) & 0xffu;
          uint2 qv = make_uint2(0u, 0u);
          if (cj != 0xffu) qv = *reinterpret_cast<const uint2*>(qh16 + r * qstride + 4 * cj);
          const uint4 a = *reinterpret_cast<const uint4*>(rec + 16 + lane * 16);
          mma16816(s2, a.x, a.y, a.z, a.w, qv.x, qv.y);
        }
        if (anyK) {
          // K outliers: their rows decode to 0 (radius code 0), so their scores are added by extra MMA
          // k-slices.  The distinct chunk positions flagged anywhere in the tile are taken four at a time
          // (lane group j <-> position c_j); A holds x * qmax / rs for the flagged (token, position) pairs,
          // split into an fp16 head and an fp16 remainder so that the product is exact to ~2^-22, and B
          // holds the query values of position c_j.  The result lands in the same accumulators and is
          // scaled with them.
          // staged entries start at the even entry index at or below the tile's first entry
          OutlSide ok_;
          ok_.init(p.K, bh, reinterpret_cast<uint2*>(const_cast<unsigned char*>(sb) + SL::kPayK));
          const uint32_t pre16 = excl_scan16(__popc(fk_tile), lane);
          uint32_t any_c = __reduce_or_sync(0xffffffffu, fk_tile);
          uint32_t fl[2], pre[2]; float kinv[2];
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            fl[nt] = __shfl_sync(0xffffffffu, fk_tile, nt * 8 + r);
            pre[nt] = __shfl_sync(0xffffffffu, pre16, nt * 8 + r) + (offk & 1u);
            kinv[nt] = fl[nt] ? __fdividef(p.qmaxf, ld.kscale(cur, nt)) : 0.f;
          }
          while (any_c) {
            int cj = -1;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int c = any_c ? __ffs(any_c) - 1 : -1;
              any_c &= any_c - 1;
              if (q == j) cj = c;
            }
            uint32_t ahi[4] = {0u, 0u, 0u, 0u}, alo[4] = {0u, 0u, 0u, 0u}, b0 = 0u, b1 = 0u;
            if (cj >= 0) {
              const uint2 qv = *reinterpret_cast<const uint2*>(qh16 + r * qstride + 4 * cj);
              b0 = qv.x; b1 = qv.y;
#pragma unroll
              for (int nt = 0; nt < 2; ++nt) {
                if ((fl[nt] >> cj) & 1u) {
                  const uint32_t rel = pre[nt] + __popc(fl[nt] & ((1u << cj) - 1u));
                  const float4 x = ok_.loadf(offk - (offk & 1u) + rel, rel <= (uint32_t)kPay ? rel : 0xffffffffu);
                  const float v0 = x.x * kinv[nt], v1 = x.y * kinv[nt], v2 = x.z * kinv[nt], v3 = x.w * kinv[nt];
                  const __half2 h01 = __floats2half2_rn(v0, v1), h23 = __floats2half2_rn(v2, v3);
                  const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
                  ahi[nt] = *reinterpret_cast<const uint32_t*>(&h01);
                  ahi[2 + nt] = *reinterpret_cast<const uint32_t*>(&h23);
                  alo[nt] = pack_half2(v0 - f01.x, v1 - f01.y);
                  alo[2 + nt] = pack_half2(v2 - f23.x, v3 - f23.y);
                }
              }
            }
            mma16816(s, ahi[0], ahi[1], ahi[2], ahi[3], b0, b1);
            mma16816(s2, alo[0], alo[1], alo[2], alo[3], b0, b1);
          }
        }
      }
#pragma unroll
      for (int x = 0; x < 4; ++x) s[x] += s2[x];

      // ---- scale, outlier scores, mask, online softmax -----------------------------------------------------
      bool grew = false;
      float mx[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        s[e] = okt[0] ? s[e] * ksc[0] : -INFINITY;
        s[2 + e] = okt[1] ? s[2 + e] * ksc[1] : -INFINITY;
        float m = fmaxf(s[e], s[2 + e]);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
        mx[e] = m;
        grew |= m > m_run[e];
      }
      if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float m_new = fmaxf(m_run[e], mx[e]);
          const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_run[e] - m_new);
          m_run[e] = m_new;
          l_run[e] *= alpha;
#pragma unroll
          for (int i = 0; i < NOT; ++i) { o[i][e] *= alpha; o[i][2 + e] *= alpha; }
        }
      }
      // P goes to the tensor cores as fp16(p * rs_V / qmax); the weights summed into l are those rounded products
      // divided by the same scale again, so numerator and denominator of the output use one set of weights and the
      // rounding of P cancels instead of adding 2^-11 of relative error to an output that a single key dominates.
      uint32_t pb[2];
      {
        float pe[4];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float m_use = m_run[e] == -INFINITY ? 0.f : m_run[e];
          pe[e] = fast_exp2(s[e] - m_use);
          pe[2 + e] = fast_exp2(s[2 + e] - m_use);
        }
        const __half2 h0 = __floats2half2_rn(pe[0] * vsc[0], pe[1] * vsc[0]);
        const __half2 h1 = __floats2half2_rn(pe[2] * vsc[1], pe[3] * vsc[1]);
        float iv0 = 0.f, iv1 = 0.f;
        if (vsc[0] > 0.f) asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(iv0) : "f"(vsc[0]));
        if (vsc[1] > 0.f) asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(iv1) : "f"(vsc[1]));
        const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
        // (a token whose scale is zero -- an all-zero V row under fp16 scales -- adds nothing to the numerator but
        //  keeps its weight in the denominator; a masked token has weight 0 already)
        l_run[0] += (vsc[0] > 0.f ? f0.x * iv0 : pe[0]) + (vsc[1] > 0.f ? f1.x * iv1 : pe[2]);
        l_run[1] += (vsc[0] > 0.f ? f0.y * iv0 : pe[1]) + (vsc[1] > 0.f ? f1.y * iv1 : pe[3]);
        pb[0] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&h0));
        pb[1] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&h1));
      }

      // ---- O^T += V^T P^T -------------------------------------------------------------------------------------
      auto v_side = [&](auto patch_) {
        constexpr bool PATCH = decltype(patch_)::value;
        // flag words, payload positions and inverse scales of this lane's four tokens (patch path only)
        uint32_t vfl[4] = {0, 0, 0, 0}, vpre[4] = {0, 0, 0, 0};
        float vinv[4] = {0.f, 0.f, 0.f, 0.f};
        OutlSide ov_;
        if constexpr (PATCH) {
          ov_.init(p.V, bh, reinterpret_cast<uint2*>(const_cast<unsigned char*>(sb) + SL::kPayV));
          const uint32_t ex = excl_scan16(__popc(fv_tile), lane);
          const float i0 = __fdividef(p.qmaxf, ld.vscale(cur, 0)), i1 = __fdividef(p.qmaxf, ld.vscale(cur, 1));
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int tl = 2 * j + (i & 1) + (i >> 1) * 8;
            vfl[i] = __shfl_sync(0xffffffffu, fv_tile, tl);
            vpre[i] = __shfl_sync(0xffffffffu, ex, tl);
            vinv[i] = __shfl_sync(0xffffffffu, (i >> 1) ? i1 : i0, (tl & 7) * 4);   // token tl's scale lives where r == tl & 7
          }
        }
        static_for<0, NVG>([&](auto g_) {
          constexpr int g = decltype(g_)::value;
          uint32_t lo[4], hi[4];
          static_for<0, 4>([&](auto i_) {
            constexpr int i = decltype(i_)::value;
            uint32_t idx; __half2 rr;
            ld.template voff<i, g>(cur, idx, rr);
            const uint2 cw = *reinterpret_cast<const uint2*>(tblV + idx);
            lo[i] = hmul2_u32(cw.x, rr);
            hi[i] = hmul2_u32(cw.y, rr);
            if constexpr (PATCH) {
              const int c = r * NVG + g;
              if (c < N && ((vfl[i] >> c) & 1u)) {
                const uint32_t rel = vpre[i] + __popc(vfl[i] & ((1u << c) - 1u));
                const uint32_t skew = offv & 1u;
                ov_.load(offv + rel, rel + skew <= (uint32_t)kPay ? rel + skew : 0xffffffffu, vinv[i], lo[i], hi[i]);
              }
            }
          });
          const uint32_t a0 = __byte_perm(lo[0], lo[1], 0x5410), a1 = __byte_perm(lo[0], lo[1], 0x7632);
          const uint32_t a2 = __byte_perm(lo[2], lo[3], 0x5410), a3 = __byte_perm(lo[2], lo[3], 0x7632);
          const uint32_t c0 = __byte_perm(hi[0], hi[1], 0x5410), c1 = __byte_perm(hi[0], hi[1], 0x7632);
          const uint32_t c2 = __byte_perm(hi[2], hi[3], 0x5410), c3 = __byte_perm(hi[2], hi[3], 0x7632);
          mma16816(o[2 * g], a0, a1, a2, a3, pb[0], pb[1]);
          mma16816(o[2 * g + 1], c0, c1, c2, c3, pb[0], pb[1]);
        });
      };
      if (OUTL && anyV) v_side(std::true_type{});
      else v_side(std::false_type{});
      __syncwarp();   // every lane is done with the stage before lane 0 refills it
    }
    if (failed && !drained) {
      drained = true;
      // drain: the copies still in flight for this warp land in its own buffers; wait for them (bounded)
      // so that no copy is outstanding when the CTA exits
      for (int k = 0; k < kStages; ++k) {
        uint32_t spins = 0;
        while (!mbar_try_wait(bar0 + 8 * ((it + k) % kStages), ((it + k) / kStages) & 1u) && ++spins < kWaitLimit) {}
      }
    }

    // ---- warp mode: this warp's partial of the unit goes to its own slot (part, warp); the merge kernel skips the
    // empty ones by their header -----------------------------------------------------------------------------------
    if (wm) {
      const int n_parts = p.P * NW;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float l = l_run[e];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        const int g = 2 * j + e;
        if (g >= p.G) continue;
        const int64_t row = ((int64_t)b * p.Hq + h * p.G + g) * p.Tq + tq;
        float* dst = p.partials + (row * n_parts + part * NW + warp) * (4 * N + 2);
        if (n_my > 0) {
#pragma unroll
          for (int i = 0; i < NOT; ++i) {
            const int chunk = r * NVG + (i >> 1);
            if (chunk < N) {
              dst[4 * chunk + 2 * (i & 1)] = o[i][e];
              dst[4 * chunk + 2 * (i & 1) + 1] = o[i][2 + e];
            }
          }
        }
        if (r == 0) { dst[4 * N] = m_run[e]; dst[4 * N + 1] = l; }
      }
      continue;
    }

    // ---- one partial per (CTA, unit, head): the warps' results are merged in shared memory ---------------------
    // The rings are idle between units (every issued tile was consumed), so their memory holds the warps'
    // partials [warp][head][d + 2] for the merge.  A warp that gave up on a wait takes the whole CTA out here.
    if (__syncthreads_or(failed ? 1 : 0)) break;
    constexpr int PD = 4 * N + 2;
    float* mp = reinterpret_cast<float*>(warp_area);
    {
      float* mine = mp + warp * NHEADS * PD;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float l = l_run[e];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        float* dst = mine + (2 * j + e) * PD;
#pragma unroll
        for (int i = 0; i < NOT; ++i) {
          const int chunk = r * NVG + (i >> 1);
          if (chunk < N) {
            dst[4 * chunk + 2 * (i & 1)] = o[i][e];
            dst[4 * chunk + 2 * (i & 1) + 1] = o[i][2 + e];
          }
        }
        if (r == 0) { dst[4 * N] = m_run[e]; dst[4 * N + 1] = l; }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.G * (4 * N); i += NW * 32) {
      const int g = i / (4 * N), x = i - g * (4 * N);
      const float* col = mp + g * PD;
      float m_star = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) m_star = fmaxf(m_star, col[w * NHEADS * PD + 4 * N]);
      const float m_use = m_star == -INFINITY ? 0.f : m_star;
      float acc = 0.f, l_star = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float wgt = fast_exp2(col[w * NHEADS * PD + 4 * N] - m_use);   // 0 for a warp that saw no key
        acc = fmaf(col[w * NHEADS * PD + x], wgt, acc);
        l_star = fmaf(col[w * NHEADS * PD + 4 * N + 1], wgt, l_star);
      }
      const int64_t row = ((int64_t)b * p.Hq + h * p.G + g) * p.Tq + tq;
      float* dst = p.partials + (row * p.P + part) * PD;
      dst[x] = acc;
      if (x == 0) { dst[4 * N] = m_star; dst[4 * N + 1] = l_star; }
    }
    __syncthreads();   // the merge is done with the ring memory before the next unit's copies land in it
  }
}

}  // namespace attn
}  // namespace hqmq
