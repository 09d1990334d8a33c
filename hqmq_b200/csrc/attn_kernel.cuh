// Fused decode attention over the compressed KV cache (sm_100a): kernel body and loaders.
//
// Work decomposition.  A "unit" is one (KV head, batch, query position); its keys are walked in
// 16-token tiles.  The tiles of all units form one flat sequence that is cut into equal pieces,
// one per CTA, so every SM gets the same amount of work whatever the shape; a CTA's piece is a
// list of segments (unit, tile range).  All G = H_q/H_kv query heads of a unit share every
// decoded key/value.  Within a segment the CTA's warps take tiles round-robin:
//   K side  S^T = K Q^T on tensor cores (m16n8k16, fp16 in, fp32 accumulate) with the 16 tokens of
//           the tile as the M rows and the (up to 8) query heads as the N columns, so no row of
//           the instruction is padding.  The head dimension is permuted so that the codeword a
//           lane gathers from the shared-memory table (4 fp16) is exactly its share of the A
//           fragment; it is scaled by the integer radius code on the way.  The per-token scale
//           rs/qmax and the softmax scale are applied to the fp32 scores.
//   softmax online (running max / sum per query head, exp2 domain); the accumulators are only
//           rescaled when some head's maximum actually grew.
//   V side  O^T += V^T P^T with 16 head-dims as M rows and the heads as N columns: gather +
//           radius, byte-permute token pairs into A fragments; P is transposed between the two
//           products with movmatrix; the per-token V scale is folded into P.
// Every warp writes an un-normalised partial (o[d], m, l) per query head and segment; a second
// kernel merges the partials of a unit (and is also what merges partials gathered from other GPUs).
#pragma once
#include <math.h>
#include <string.h>

#include <type_traits>

#include "common.cuh"

namespace hqmq {
namespace attn {

constexpr int kTile = 16;
#ifndef HQMQ_FAST_WARPS_OUTL
#define HQMQ_FAST_WARPS_OUTL 16
#endif
#ifndef HQMQ_FAST_WARPS
#define HQMQ_FAST_WARPS 16
#endif
constexpr int kFastWarps = HQMQ_FAST_WARPS, kFastWarpsOutl = HQMQ_FAST_WARPS_OUTL, kSlowWarps = 4;   // warps per CTA of the kernel families
constexpr int kStage = 64;   // outlier payload entries staged per tile and tensor
static_assert(kTile == HQMQ_OUT_BLOCK, "one outlier-offset entry per KV tile");

struct AttnParams {
  int B, Hq, Hkv, G, Tq, Tkv, d;
  int causal, window;
  float sscale;  // softmax_scale * log2(e) / qmax
  float qscale;  // softmax_scale * log2(e)
  float vscale;  // 1 / qmax
  float qmaxf;
  int nw;        // warps per CTA
  int rep_log2;  // the codeword tables are replicated 2^rep_log2 times, interleaved entry by entry
  int repv_log2;      // ring kernels: replication of the V table (rep_log2 is then the K table's)
  int ring_stages;    // ring kernels: stages of the CTA-wide staging ring
  int merge_slots;    // ring kernels: warps whose partials are merged per round at the end of a unit
  int unit_hfast;     // ring kernels: units are numbered with the KV head running fastest (u = (b, tq) * H_kv + h)
  int warp_units;     // staged kernels: the warps of a CTA walk through the units independently (one partial per warp)
  // flat tile space: units * tpu_v virtual tiles, L per CTA; a unit is touched by at most P CTAs
  int units, tpu_v, L, P;
  const void* Q; int q_dtype; int64_t qs_b, qs_h, qs_t;
  float* partials;  // [row][P * nw][d+2]
  int layout;       // 0 native, 1 reference tuple
  int ib;           // index bits of a field (native: idx_bits; reference: 16)
  int table_rows;   // codewords per head in the shared-memory tables
  hqmq_packed K, V;
  const uint16_t* tblK; const uint16_t* tblV;
  hqmq_ref_packed Kr, Vr;
  const void* jK; const void* jV; int j_dtype;
  uint32_t* status;   // a kernel that gave up on a bounded wait stores `epoch` here; the merge kernel then emits NaN
  uint32_t epoch;
  // ring kernels: the merge over the CTAs of a unit is done by the last of them to finish (one ticket per unit)
  uint32_t* tickets;  // [units], zero at launch
  void* O; int o_dtype; int64_t os_b, os_h, os_t;
  float* merged;      // partials_only: one merged (o[d], m, l) per row instead of O
};

// A ring kernel (attn_ring.cu) and the bytes of one of its stages.
struct RingKernelInfo { const void* fn; size_t stage_bytes; int warps; };   // warps: consumers (one more warp produces)

// Key range [beg, end) of query position tq.  causal 1: the reference's top-left aligned mask (query i sees keys
// 0..i); causal 2: bottom-right aligned (the Tq queries are the LAST Tq positions of the Tkv keys: query i sees keys
// 0..Tkv - Tq + i, a prompt chunk attending over a cache that already holds it).
__host__ __device__ inline void key_range(int Tkv, int Tq, int causal, int window, int tq, int& beg, int& end) {
  end = causal == 1 ? (tq + 1 < Tkv ? tq + 1 : Tkv) : causal == 2 ? (Tkv - Tq + tq + 1 > 0 ? Tkv - Tq + tq + 1 : 0) : Tkv;
  if (end > Tkv) end = Tkv;
  beg = window > 0 ? (end - window > 0 ? end - window : 0) : 0;
}

__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Transpose an 8x8 matrix of 16-bit elements held one row-pair per lane (the C-fragment layout of
// one half of an accumulator, packed to half2) into the B-fragment layout.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, __half2 r) {
  __half2 v = __hmul2(*reinterpret_cast<__half2*>(&a), r);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Integer radius code (< 1024) as half2 (r, r): 0x6400 | r is the half 1024 + r.
__device__ __forceinline__ __half2 radius_half2(uint32_t rq) {
  uint32_t bits = 0x64006400u | (rq * 0x10001u);
  return __hsub2(*reinterpret_cast<__half2*>(&bits), __float2half2_rn(1024.f));
}

template <int N>
struct Geo {
  static constexpr int NKS = N / 4;        // 16-wide k slices of the head dimension
  static constexpr int NVG = (N + 7) / 8;  // chunks per lane row on the V side
  static constexpr int NOT = NVG * 4;      // 8-wide output tiles (padded)
};

// Words a lane must read to cover `L` bits starting at bit j*L (j = 0..lanes-1) of a row.
constexpr int span_words(int L, int lanes) {
  int m = 0;
  for (int j = 0; j < lanes; ++j) {
    int w = (((j * L) & 31) + L + 31) / 32;
    if (w > m) m = w;
  }
  return m;
}

// ---- loaders ---------------------------------------------------------------------------------------
// Raw data of one 16-token tile for one lane.  Lane (j = lane & 3, r = lane >> 2):
//   K side: tokens nt*8 + r (nt = 0,1), chunks j*NKS .. j*NKS + NKS-1
//   V side: tokens {2j, 2j+1, 2j+8, 2j+9}, chunks r*NVG .. r*NVG + NVG-1
//   scales of tokens r and r+8 for K and for V.

// Native layout, compile-time field layout (IB index bits + RB radius bits): rows are read as raw
// words and fields are cut in registers.
template <int N, int IB, int RB, bool FOLD>
struct FastLoader {
  static constexpr int CB = IB + RB;
  static constexpr int NKS = Geo<N>::NKS, NVG = Geo<N>::NVG;
  static constexpr int LK = NKS * CB, LV = NVG * CB;
  static constexpr int KW = span_words(LK, 4), VW = span_words(LV, 8);
  struct Raw { uint32_t kw[2][KW + 1]; uint32_t vw[4][VW + 1]; uint16_t rsk[2], rsv[2]; };
  const uint8_t* kc; const uint8_t* vc; const uint16_t* krs; const uint16_t* vrs;
  int row_bytes, row_words, j, r, sdt;

  __device__ __forceinline__ void init(const AttnParams& p, int b, int h, int lane) {
    const int64_t bh = (int64_t)b * p.Hkv + h;
    row_bytes = p.K.row_bytes; row_words = row_bytes >> 2;
    kc = p.K.codes + bh * p.K.T_cap * row_bytes;
    vc = p.V.codes + bh * p.V.T_cap * row_bytes;
    krs = reinterpret_cast<const uint16_t*>(p.K.rs) + bh * p.K.T_cap;
    vrs = reinterpret_cast<const uint16_t*>(p.V.rs) + bh * p.V.T_cap;
    j = lane & 3; r = lane >> 2; sdt = p.K.scale_dtype;
  }
  template <int W, int L>
  __device__ __forceinline__ void load_span(uint32_t* dst, const uint8_t* row, int part, bool ok) const {
    const uint32_t* rp = reinterpret_cast<const uint32_t*>(row);
    const int sb = part * L, w0 = sb >> 5, sh = sb & 31;
    if constexpr (L % 128 == 0) {
#pragma unroll
      for (int i = 0; i < W; i += 4) {
        uint4 v = ok ? *reinterpret_cast<const uint4*>(rp + w0 + i) : make_uint4(0, 0, 0, 0);
        dst[i] = v.x; dst[i + 1] = v.y; dst[i + 2] = v.z; dst[i + 3] = v.w;
      }
      dst[W] = 0;
    } else if constexpr (L % 64 == 0) {
#pragma unroll
      for (int i = 0; i < W; i += 2) {
        uint2 v = ok ? *reinterpret_cast<const uint2*>(rp + w0 + i) : make_uint2(0, 0);
        dst[i] = v.x; dst[i + 1] = v.y;
      }
      dst[W] = 0;
    } else if constexpr (L % 32 == 0) {
#pragma unroll
      for (int i = 0; i < W; ++i) dst[i] = ok ? rp[w0 + i] : 0u;
      dst[W] = 0;
    } else {
      uint32_t t[W + 1];
#pragma unroll
      for (int i = 0; i < W; ++i) t[i] = ok ? rp[min(w0 + i, row_words - 1)] : 0u;
      t[W] = 0;
#pragma unroll
      for (int i = 0; i < W; ++i) dst[i] = __funnelshift_r(t[i], t[i + 1], sh);
      dst[W] = 0;
    }
  }
  __device__ __forceinline__ void fetch(Raw& raw, int tile, int t_end) const {
    const int t0 = tile * kTile;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int t = t0 + nt * 8 + r;
      load_span<KW, LK>(raw.kw[nt], kc + (int64_t)t * row_bytes, j, t < t_end);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = t0 + 2 * j + (i & 1) + (i >> 1) * 8;
      load_span<VW, LV>(raw.vw[i], vc + (int64_t)t * row_bytes, r, t < t_end);
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int t = t0 + nt * 8 + r;
      raw.rsk[nt] = krs[t];
      raw.rsv[nt] = vrs[t];
    }
  }
  // Field F -> codeword table index and radius as half2 (r, r).
  // FOLD: the table is SIGN-FOLDED.  The lowest bit of a native index is the sign of the axis unit u
  // (u = 2*axis + sign) and the codeword of -u is exactly minus the codeword of +u, so the table keeps only
  // the even entries (half the shared memory, which buys twice the replication against bank conflicts) and
  // the sign goes into the radius, at the price of a few more instructions per gather.
  template <int F>
  static __device__ __forceinline__ void cut(const uint32_t* w, uint32_t& idx, __half2& rr) {
    constexpr int bit = F * CB, a = bit >> 5, s = bit & 31;
    if constexpr (CB == 16) {
      // two fields per word: both radii come out of one subtraction
      const uint32_t word = w[a];
      idx = FOLD ? (word >> (s + 1)) & ((1u << (IB - 1)) - 1u) : (word >> s) & ((1u << IB) - 1u);
      uint32_t bits = ((word >> IB) & (((1u << RB) - 1u) * 0x10001u)) | 0x64006400u;
      const __half2 pair = __hsub2(*reinterpret_cast<__half2*>(&bits), __float2half2_rn(1024.f));
      uint32_t pu = *reinterpret_cast<const uint32_t*>(&pair);
      // sign bits of both fields (bits 0 and 16 of the word) into the sign bits of the two halves
      if constexpr (FOLD) pu ^= (word << 15) & 0x80008000u;
      // broadcast one half to both lanes (the compiler folds this into the multiply's operand selector)
      const __half2 p2 = *reinterpret_cast<const __half2*>(&pu);
      rr = s == 0 ? __low2half2(p2) : __high2half2(p2);
    } else {
      uint32_t v = (s + CB > 32) ? __funnelshift_r(w[a], w[a + 1], s) : (w[a] >> s);
      const __half2 r2 = radius_half2((v >> IB) & ((1u << RB) - 1u));
      if constexpr (FOLD) {
        idx = (v & ((1u << IB) - 1u)) >> 1;
        const uint32_t ru = *reinterpret_cast<const uint32_t*>(&r2) ^ ((0u - (v & 1u)) & 0x80008000u);
        rr = *reinterpret_cast<const __half2*>(&ru);
      } else {
        idx = v & ((1u << IB) - 1u);
        rr = r2;
      }
    }
  }
  template <int NT, int KS> __device__ __forceinline__ void kfield(const Raw& raw, uint32_t& idx, __half2& rr) const {
    cut<KS>(raw.kw[NT], idx, rr);
  }
  template <int I, int GG> __device__ __forceinline__ void vfield(const Raw& raw, uint32_t& idx, __half2& rr) const {
    cut<GG>(raw.vw[I], idx, rr);
    if constexpr (N % 8 != 0) { if (r * NVG + GG >= N) { idx = 0; rr = __float2half2_rn(0.f); } }
  }
  // The same, but straight to the byte offset of the codeword in a table whose entries are `stride` bytes
  // apart (plus this lane's replica offset).  With two 16-bit fields per word the shifts are done by the
  // multiplier: offset = hi32(masked field * (stride << 16)), radius pair = hi32(masked nibbles << 20), which
  // keeps them off the half-rate shift/logic pipe.  Used by the full-table (outlier) kernels only: with the
  // sign-folded table the same change measured 13 % slower.
  uint32_t mul_lo, mul_hi, lane_off;   // stride (halved for a sign-folded table), the same << 16, replica offset
  __device__ __forceinline__ void set_table(uint32_t rstride, uint32_t lane_off_) {
    mul_lo = FOLD ? rstride >> 1 : rstride; mul_hi = mul_lo << 16; lane_off = lane_off_;
  }
  static __device__ __forceinline__ uint32_t mad_hi(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.hi.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
  }
  template <int F>
  __device__ __forceinline__ void cut_off(const uint32_t* w, uint32_t& off, __half2& rr) const {
    if constexpr (CB == 16 && !FOLD) {
      constexpr int bit = F * CB, a = bit >> 5, s = bit & 31;
      const uint32_t word = w[a];
      constexpr uint32_t imask = (1u << IB) - 1u;
      if constexpr (s == 0) off = (word & imask) * mul_lo + lane_off;
      else off = mad_hi(word & (imask << 16), mul_hi, lane_off);
      constexpr uint32_t rmask = (((1u << RB) - 1u) << IB) * 0x10001u;
      uint32_t bits = mad_hi(word & rmask, 1u << (32 - IB), 0x64006400u);
      const __half2 pair = __hsub2(*reinterpret_cast<__half2*>(&bits), __float2half2_rn(1024.f));
      rr = s == 0 ? __low2half2(pair) : __high2half2(pair);
    } else {
      uint32_t idx;
      cut<F>(w, idx, rr);
      off = idx * (FOLD ? mul_lo * 2u : mul_lo) + lane_off;
    }
  }
  template <int NT, int KS> __device__ __forceinline__ void koff(const Raw& raw, uint32_t& off, __half2& rr) const {
    cut_off<KS>(raw.kw[NT], off, rr);
  }
  template <int I, int GG> __device__ __forceinline__ void voff(const Raw& raw, uint32_t& off, __half2& rr) const {
    cut_off<GG>(raw.vw[I], off, rr);
    if constexpr (N % 8 != 0) { if (r * NVG + GG >= N) { off = lane_off; rr = __float2half2_rn(0.f); } }
  }
  // scale of token nt*8 + r
  __device__ __forceinline__ float kscale(const Raw& raw, int nt) const { return bits16_to_float(raw.rsk[nt], sdt); }
  __device__ __forceinline__ float vscale(const Raw& raw, int nt) const { return bits16_to_float(raw.rsv[nt], sdt); }
};

// Any field width, native or reference layout: fields are extracted one by one at load time.
template <int N>
struct SlowLoader {
  static constexpr int NKS = Geo<N>::NKS, NVG = Geo<N>::NVG;
  struct Raw { uint32_t kf[2][NKS]; uint32_t vf[4][NVG]; float rsk[2], rsv[2]; };
  const AttnParams* pp; int b, h, j, r;
  __device__ __forceinline__ void init(const AttnParams& p_, int b_, int h_, int lane) {
    pp = &p_; b = b_; h = h_; j = lane & 3; r = lane >> 2;
  }
  __device__ __forceinline__ uint32_t field(const hqmq_packed& pk, const hqmq_ref_packed& rf, int t, int c) const {
    const AttnParams& p = *pp;
    if (p.layout == 0) {
      const int cb = p.ib + pk.radius_bits;
      const int64_t row = ((int64_t)b * p.Hkv + h) * pk.T_cap + t;
      return row_field(reinterpret_cast<const uint32_t*>(pk.codes + row * pk.row_bytes), c, cb);
    }
    long long k = load_int(rf.idx, b * rf.idx_stride[0] + h * rf.idx_stride[1] + t * rf.idx_stride[2] + c, rf.idx_dtype);
    k = k < 0 ? 0 : (k >= p.table_rows ? p.table_rows - 1 : k);
    long long q = load_int(rf.rq, b * rf.rq_stride[0] + h * rf.rq_stride[1] + t * rf.rq_stride[2] + c, rf.rq_dtype);
    q = q < 0 ? 0 : (q > 1023 ? 1023 : q);
    return (uint32_t)k | ((uint32_t)q << 16);
  }
  __device__ __forceinline__ float rscale(const hqmq_packed& pk, const hqmq_ref_packed& rf, int t) const {
    const AttnParams& p = *pp;
    if (p.layout == 0) return load_scale(pk, ((int64_t)b * p.Hkv + h) * pk.T_cap + t);
    return load_float(rf.rs, b * rf.rs_stride[0] + h * rf.rs_stride[1] + t, rf.rs_dtype);
  }
  __device__ __forceinline__ void fetch(Raw& raw, int tile, int t_end) const {
    const AttnParams& p = *pp;
    const int t0 = tile * kTile;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int t = t0 + nt * 8 + r;
#pragma unroll
      for (int ks = 0; ks < NKS; ++ks) raw.kf[nt][ks] = t < t_end ? field(p.K, p.Kr, t, j * NKS + ks) : 0u;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = t0 + 2 * j + (i & 1) + (i >> 1) * 8;
#pragma unroll
      for (int g = 0; g < NVG; ++g) {
        const int c = r * NVG + g;
        raw.vf[i][g] = (t < t_end && c < N) ? field(p.V, p.Vr, t, c) : 0u;
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int t = t0 + nt * 8 + r;
      raw.rsk[nt] = t < t_end ? rscale(p.K, p.Kr, t) : 0.f;
      raw.rsv[nt] = t < t_end ? rscale(p.V, p.Vr, t) : 0.f;
    }
  }
  __device__ __forceinline__ void split(uint32_t f, uint32_t& idx, __half2& rr) const {
    idx = f & ((1u << pp->ib) - 1u);
    rr = radius_half2(f >> pp->ib);
  }
  template <int NT, int KS> __device__ __forceinline__ void kfield(const Raw& raw, uint32_t& idx, __half2& rr) const {
    split(raw.kf[NT][KS], idx, rr);
  }
  template <int I, int GG> __device__ __forceinline__ void vfield(const Raw& raw, uint32_t& idx, __half2& rr) const {
    split(raw.vf[I][GG], idx, rr);
  }
  __device__ __forceinline__ float kscale(const Raw& raw, int nt) const { return raw.rsk[nt]; }
  __device__ __forceinline__ float vscale(const Raw& raw, int nt) const { return raw.rsv[nt]; }
};

// Two packed 16-bit floats (fp16 or bf16) to fp32 with one uniform branch.
__device__ __forceinline__ float2 pair16_to_float2(uint32_t v, int dtype) {
  if (dtype == HQMQ_BF16) return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

// ---- Med3x outliers ----------------------------------------------------------------------------------
// Flagged chunks keep their original 4 values in a side buffer, in (token, chunk) order, with one
// offset per 16-token tile, so a tile's entries are one contiguous range; their radius code in the
// packed row is 0, so the tensor-core path contributes nothing for them.
//   K: after S^T is accumulated, the lanes walk the tile's flagged chunks and add <q, x> in fp32 to the
//      scores (exact whatever the magnitude of the outlier).
//   V: the decoded fragment is overwritten with x * qmax / rs: the token's scale rs is its largest chunk
//      norm, flagged chunks included, so the patched value never exceeds qmax and cannot overflow fp16.
// The first kStage entries of a tile are prefetched a tile ahead and staged in shared memory; anything
// beyond (or an fp32 side buffer) is read from global memory in place.
struct OutlRaw { uint32_t fk, fv, offk, offv; uint2 pk[kStage / 32], pv[kStage / 32]; };

struct OutlSide {
  const uint32_t* flags; const uint32_t* off; const unsigned char* vals; int dtype; uint2* stage;
  uint32_t cap;   // entries the (b,h) side buffer holds; an entry at or beyond it was dropped by the encoder and reads as 0
  __device__ __forceinline__ void init(const hqmq_packed& pk, int64_t bh, uint2* stage_) {
    cap = (uint32_t)pk.out_cap;
    flags = pk.flags ? pk.flags + bh * pk.T_cap : nullptr;
    off = pk.flags ? pk.out_off + bh * (pk.T_cap / HQMQ_OUT_BLOCK + 1) : nullptr;
    dtype = pk.out_dtype;
    vals = reinterpret_cast<const unsigned char*>(pk.out_vals) + bh * pk.out_cap * 4 * (dtype == HQMQ_F32 ? 4 : 2);
    stage = stage_;
  }
  // original values of payload entry `pos` (tile-relative index `rel`)
  __device__ __forceinline__ float4 loadf(uint32_t pos, uint32_t rel) const {
    if (pos >= cap) return make_float4(0.f, 0.f, 0.f, 0.f);
    if (dtype == HQMQ_F32) return *reinterpret_cast<const float4*>(vals + (int64_t)pos * 16);
    const uint2 v = rel < (uint32_t)kStage ? stage[rel] : *reinterpret_cast<const uint2*>(vals + (int64_t)pos * 8);
    const float2 a = pair16_to_float2(v.x, dtype), b = pair16_to_float2(v.y, dtype);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  // the same scaled by `inv`, as two half2 registers
  __device__ __forceinline__ void load(uint32_t pos, uint32_t rel, float inv, uint32_t& lo, uint32_t& hi) const {
    float x0, x1, x2, x3;
    if (pos >= cap) {
      x0 = x1 = x2 = x3 = 0.f;
    } else if (dtype == HQMQ_F32) {
      const float4 v = *reinterpret_cast<const float4*>(vals + (int64_t)pos * 16);
      x0 = v.x; x1 = v.y; x2 = v.z; x3 = v.w;
    } else {
      const uint2 v = rel < (uint32_t)kStage ? stage[rel] : *reinterpret_cast<const uint2*>(vals + (int64_t)pos * 8);
      const float2 a = pair16_to_float2(v.x, dtype), b = pair16_to_float2(v.y, dtype);
      x0 = a.x; x1 = a.y; x2 = b.x; x3 = b.y;
    }
    lo = pack_half2(x0 * inv, x1 * inv);
    hi = pack_half2(x2 * inv, x3 * inv);
  }
};

// Exclusive prefix sum of v over lanes 0..15 (lanes >= 16 hold 0).
__device__ __forceinline__ uint32_t excl_scan16(uint32_t v, int lane) {
  uint32_t x = v;
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  return x - v;
}

template <int I, int End, class F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < End) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, End>(f);
  }
}

// Loader: FastLoader<N, IB, RB> or SlowLoader<N>.  NW: warps per CTA.  OUTL: merge Med3x outliers.
// WIDE: 8 < G <= 16.
template <int N, class Loader, int NW, bool OUTL, bool WIDE>
__device__ __forceinline__ void attn_decode_body(const AttnParams& p) {
  using G_ = Geo<N>;
  constexpr int NKS = G_::NKS, NVG = G_::NVG, NOT = 2 * G_::NVG;   // NOT: 16-row tiles of O^T
  constexpr int NH = WIDE ? 2 : 1;   // 8-wide head tiles
  constexpr int NHEADS = 8 * NH;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t rstride = 8u << p.rep_log2;                       // bytes between consecutive codewords
  const size_t tbl_bytes = (size_t)p.table_rows * rstride;
  unsigned char* tblK = smem_raw;
  unsigned char* tblV = smem_raw + tbl_bytes;
  float* qf32 = reinterpret_cast<float*>(smem_raw + 2 * tbl_bytes);                // [NHEADS][d]   (OUTL)
  unsigned char* warp_base = reinterpret_cast<unsigned char*>(qf32 + NHEADS * p.d); // per warp      (OUTL)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = lane & 3, r = lane >> 2;
  const uint32_t lane_off = (uint32_t)(lane & ((1 << p.rep_log2) - 1)) * 8u;       // this lane's replica
  uint2* stageK = reinterpret_cast<uint2*>(warp_base + (size_t)warp * (2 * kStage * 8 + 16 * NHEADS * 4));
  uint2* stageV = stageK + kStage;
  float* dS = reinterpret_cast<float*>(stageV + kStage);                            // [16 tokens][NHEADS]
  const int64_t flat_lo = (int64_t)blockIdx.x * p.L;
  const int64_t flat_total = (int64_t)p.units * p.tpu_v;
  const int64_t flat_hi = flat_lo + p.L < flat_total ? flat_lo + p.L : flat_total;
  const int upb = p.B * p.Tq;   // units per KV head
  int cur_h = -1;

  for (int u = (int)(flat_lo / p.tpu_v); (int64_t)u * p.tpu_v < flat_hi; ++u) {
    const int h = u / upb, bt = u - h * upb;
    const int b = bt / p.Tq, tq = bt - b * p.Tq;
    // ---- codeword tables of this KV head into shared memory (fp16 x 4 per entry, replicated) ---------
    if (h != cur_h || OUTL) __syncthreads();
    if (h != cur_h) {
      const int reps = 1 << p.rep_log2;
      for (int i = threadIdx.x; i < p.table_rows; i += NW * 32) {
        uint2 ek, ev;
        if (p.layout == 0) {
          ek = (reinterpret_cast<const uint2*>(p.tblK) + (int64_t)h * p.table_rows)[i];
          ev = (reinterpret_cast<const uint2*>(p.tblV) + (int64_t)h * p.table_rows)[i];
        } else {
          const int64_t base = ((int64_t)h * p.table_rows + i) * 4;
          ek = make_uint2(pack_half2(load_float(p.jK, base, p.j_dtype), load_float(p.jK, base + 1, p.j_dtype)),
                          pack_half2(load_float(p.jK, base + 2, p.j_dtype), load_float(p.jK, base + 3, p.j_dtype)));
          ev = make_uint2(pack_half2(load_float(p.jV, base, p.j_dtype), load_float(p.jV, base + 1, p.j_dtype)),
                          pack_half2(load_float(p.jV, base + 2, p.j_dtype), load_float(p.jV, base + 3, p.j_dtype)));
        }
        uint2* dk = reinterpret_cast<uint2*>(tblK + (size_t)i * rstride);
        uint2* dv = reinterpret_cast<uint2*>(tblV + (size_t)i * rstride);
        for (int q = 0; q < reps; ++q) { dk[q] = ek; dv[q] = ev; }
      }
      cur_h = h;
    }
    if constexpr (OUTL) {
      // queries of this unit in fp32 for the K outlier correction
      for (int i = threadIdx.x; i < NHEADS * p.d; i += NW * 32) {
        const int g = i / p.d, x = i - g * p.d;
        qf32[i] = g < p.G ? load_float(p.Q, (int64_t)b * p.qs_b + (int64_t)tq * p.qs_t + (int64_t)(h * p.G + g) * p.qs_h + x,
                                       p.q_dtype) : 0.f;
      }
    }
    __syncthreads();

    // ---- this CTA's tiles of the unit ----------------------------------------------------------------
    int t_beg, t_end;
    key_range(p.Tkv, p.Tq, p.causal, p.window, tq, t_beg, t_end);
    const int tile_lo = t_beg / kTile, tile_hi = (t_end + kTile - 1) / kTile;
    const int64_t ubase = (int64_t)u * p.tpu_v;
    const int rel_lo = (int)(flat_lo > ubase ? flat_lo - ubase : 0);
    const int rel_hi = (int)(flat_hi < ubase + p.tpu_v ? flat_hi - ubase : p.tpu_v);
    const int my_lo = tile_lo + rel_lo;
    const int my_hi = min(tile_hi, tile_lo + rel_hi);
    const int part = ((int)blockIdx.x - (int)(ubase / p.L)) * NW + warp;

    // ---- Q as B fragments: column n = r is a query head, k slots {2j,2j+1,2j+8,2j+9} = one chunk -----
    uint32_t qb[NH][NKS][2];
    {
      const int64_t q0off = (int64_t)b * p.qs_b + (int64_t)tq * p.qs_t;
#pragma unroll
      for (int nh = 0; nh < NH; ++nh) {
        const int g = r + 8 * nh;
#pragma unroll
        for (int ks = 0; ks < NKS; ++ks) {
          const int dim = 4 * (j * NKS + ks);
          float q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
          if (g < p.G) {
            const int64_t o = q0off + (int64_t)(h * p.G + g) * p.qs_h + dim;
            q0 = load_float(p.Q, o, p.q_dtype); q1 = load_float(p.Q, o + 1, p.q_dtype);
            q2 = load_float(p.Q, o + 2, p.q_dtype); q3 = load_float(p.Q, o + 3, p.q_dtype);
          }
          qb[nh][ks][0] = pack_half2(q0, q1);
          qb[nh][ks][1] = pack_half2(q2, q3);
        }
      }
    }

    // running max and sum of heads 2j, 2j+1 (+8 per extra head tile); O^T accumulators: tile mt holds
    // head-dims (rows r, r+8) x heads (2j, 2j+1)
    float m_run[NH][2], l_run[NH][2];
    float o[NH][NOT][4];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
      m_run[nh][0] = m_run[nh][1] = -INFINITY;
      l_run[nh][0] = l_run[nh][1] = 0.f;
#pragma unroll
      for (int i = 0; i < NOT; ++i) o[nh][i][0] = o[nh][i][1] = o[nh][i][2] = o[nh][i][3] = 0.f;
    }

    Loader ld;
    ld.init(p, b, h, lane);
    OutlSide ok_, ov_;
    uint32_t offk_nn = 0, offv_nn = 0, offk_nn1 = 0, offv_nn1 = 0;   // payload ranges two tiles ahead
    if constexpr (OUTL) {
      ok_.init(p.K, (int64_t)b * p.Hkv + h, stageK);
      ov_.init(p.V, (int64_t)b * p.Hkv + h, stageV);
    }
    // flags and the first staged payload entries of tile tl, given its payload ranges
    auto fetch_outl = [&](OutlRaw& oo, int tl, uint32_t k0, uint32_t k1, uint32_t v0, uint32_t v1) {
      oo.fk = oo.fv = 0; oo.offk = k0; oo.offv = v0;
      const int tt = tl * kTile + (lane & 15);
      if (lane < 16 && tt < t_end) {
        if (ok_.flags) oo.fk = ok_.flags[tt];
        if (ov_.flags) oo.fv = ov_.flags[tt];
      }
#pragma unroll
      for (int q = 0; q < kStage / 32; ++q) {
        const uint32_t e = q * 32 + lane;
        oo.pk[q] = make_uint2(0, 0); oo.pv[q] = make_uint2(0, 0);
        if (ok_.dtype != HQMQ_F32 && k0 + e < k1 && k0 + e < ok_.cap) oo.pk[q] = *reinterpret_cast<const uint2*>(ok_.vals + (int64_t)(k0 + e) * 8);
        if (ov_.dtype != HQMQ_F32 && v0 + e < v1 && v0 + e < ov_.cap) oo.pv[q] = *reinterpret_cast<const uint2*>(ov_.vals + (int64_t)(v0 + e) * 8);
      }
    };
    auto fetch_off = [&](int tl, uint32_t& k0, uint32_t& k1, uint32_t& v0, uint32_t& v1) {
      k0 = k1 = v0 = v1 = 0;
      if (tl < my_hi) {
        if (ok_.flags) { k0 = ok_.off[tl]; k1 = ok_.off[tl + 1]; }
        if (ov_.flags) { v0 = ov_.off[tl]; v1 = ov_.off[tl + 1]; }
      }
    };
    // prefetch of tile tl into (raw, oo)
    auto fetch = [&](typename Loader::Raw& raw, OutlRaw& oo, int tl) {
      ld.fetch(raw, tl, t_end);
      if constexpr (OUTL) {
        fetch_outl(oo, tl, offk_nn, offk_nn1, offv_nn, offv_nn1);
        fetch_off(tl + NW, offk_nn, offk_nn1, offv_nn, offv_nn1);
      }
    };

    // ---- one tile -------------------------------------------------------------------------------------------
    auto compute = [&](const typename Loader::Raw& cur, const OutlRaw& ocur, int tile) {
      const int t0 = tile * kTile;
      const bool edge = t0 < t_beg || t0 + kTile > t_end;
      // per-token factors of this lane's tokens r and r+8
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

      // ---- outlier bookkeeping of this tile -----------------------------------------------------------
      bool anyK = false, anyV = false;
      uint32_t vfl[4] = {0, 0, 0, 0}, vpre[4] = {0, 0, 0, 0};
      float vinv[4] = {0.f, 0.f, 0.f, 0.f};
      if constexpr (OUTL) {
        anyK = __ballot_sync(0xffffffffu, ocur.fk != 0) != 0;
        anyV = __ballot_sync(0xffffffffu, ocur.fv != 0) != 0;
        if (anyK || anyV) {
          __syncwarp();
#pragma unroll
          for (int q = 0; q < kStage / 32; ++q) {
            ok_.stage[q * 32 + lane] = ocur.pk[q];
            ov_.stage[q * 32 + lane] = ocur.pv[q];
          }
          __syncwarp();
        }
        if (anyK) {
          // Lane t < 16 owns token t (lanes 16..31 idle along).  The warp walks the distinct chunk
          // positions that are flagged anywhere in the tile (hot channels make them few); for each, the
          // query values are one broadcast read and every flagged token adds <q_g, x> for all heads.
          const uint32_t fl = ocur.fk;                       // 0 for lanes >= 16
          const uint32_t pre = excl_scan16(__popc(fl), lane);
          uint32_t any_c = fl;
#pragma unroll
          for (int o_ = 16; o_ > 0; o_ >>= 1) any_c |= __shfl_xor_sync(0xffffffffu, any_c, o_);
          float acc[NHEADS];
#pragma unroll
          for (int g = 0; g < NHEADS; ++g) acc[g] = 0.f;
          while (any_c) {
            const int c = __ffs(any_c) - 1;
            any_c &= any_c - 1;
            if ((fl >> c) & 1u) {
              const uint32_t rel = pre + __popc(fl & ((1u << c) - 1u));
              const float4 x = ok_.loadf(ocur.offk + rel, rel);
#pragma unroll
              for (int g = 0; g < NHEADS; ++g) {
                const float4 q = *reinterpret_cast<const float4*>(qf32 + g * p.d + 4 * c);
                acc[g] = fmaf(q.w, x.w, fmaf(q.z, x.z, fmaf(q.y, x.y, fmaf(q.x, x.x, acc[g]))));
              }
            }
          }
          if (lane < 16) {
#pragma unroll
            for (int g = 0; g < NHEADS; g += 4)
              *reinterpret_cast<float4*>(dS + lane * NHEADS + g) = make_float4(acc[g], acc[g + 1], acc[g + 2], acc[g + 3]);
          }
          __syncwarp();
        }
        if (anyV) {
          const uint32_t ex = excl_scan16(__popc(ocur.fv), lane);
          const float i0 = p.qmaxf / ld.vscale(cur, 0), i1 = p.qmaxf / ld.vscale(cur, 1);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int tl = 2 * j + (i & 1) + (i >> 1) * 8;
            vfl[i] = __shfl_sync(0xffffffffu, ocur.fv, tl);
            vpre[i] = __shfl_sync(0xffffffffu, ex, tl);
            // the scale of token tl lives in the lanes whose r is tl & 7
            vinv[i] = __shfl_sync(0xffffffffu, (i >> 1) ? i1 : i0, (tl & 7) * 4);
          }
        }
      }

      // ---- S^T = K Q^T: rows = tokens r, r+8; columns = heads 2j, 2j+1 -----------------------------------
      // (even and odd k slices accumulate separately so that consecutive MMAs do not depend on each other)
      float s[NH][4], s2[NH][4];
#pragma unroll
      for (int nh = 0; nh < NH; ++nh) {
        s[nh][0] = s[nh][1] = s[nh][2] = s[nh][3] = 0.f;
        s2[nh][0] = s2[nh][1] = s2[nh][2] = s2[nh][3] = 0.f;
      }
      static_for<0, NKS>([&](auto ks_) {
        constexpr int ks = decltype(ks_)::value;
        uint32_t a[4];   // a0: token r (e0,e1), a1: token r+8 (e0,e1), a2: token r (e2,e3), a3: token r+8 (e2,e3)
        static_for<0, 2>([&](auto nt_) {
          constexpr int nt = decltype(nt_)::value;
          uint32_t idx; __half2 rr;
          ld.template kfield<nt, ks>(cur, idx, rr);
          const uint2 cw = *reinterpret_cast<const uint2*>(tblK + (idx * rstride + lane_off));
          a[nt] = hmul2_u32(cw.x, rr);
          a[2 + nt] = hmul2_u32(cw.y, rr);
        });
#pragma unroll
        for (int nh = 0; nh < NH; ++nh)
          mma16816((ks & 1) ? s2[nh] : s[nh], a[0], a[1], a[2], a[3], qb[nh][ks][0], qb[nh][ks][1]);
      });
#pragma unroll
      for (int nh = 0; nh < NH; ++nh) { s[nh][0] += s2[nh][0]; s[nh][1] += s2[nh][1]; s[nh][2] += s2[nh][2]; s[nh][3] += s2[nh][3]; }

      // ---- scale, outlier scores, mask, online softmax -----------------------------------------------------
      bool grew = false;
      float mx[NH][2];
#pragma unroll
      for (int nh = 0; nh < NH; ++nh) {
        float d0[2] = {0.f, 0.f}, d1[2] = {0.f, 0.f};
        if constexpr (OUTL) {
          if (anyK) {
            const float2 u0 = *reinterpret_cast<const float2*>(dS + r * NHEADS + 8 * nh + 2 * j);
            const float2 u1 = *reinterpret_cast<const float2*>(dS + (r + 8) * NHEADS + 8 * nh + 2 * j);
            d0[0] = u0.x * p.qscale; d0[1] = u0.y * p.qscale; d1[0] = u1.x * p.qscale; d1[1] = u1.y * p.qscale;
          }
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          s[nh][e] = okt[0] ? fmaf(s[nh][e], ksc[0], d0[e]) : -INFINITY;          // token r
          s[nh][2 + e] = okt[1] ? fmaf(s[nh][2 + e], ksc[1], d1[e]) : -INFINITY;  // token r+8
          float m = fmaxf(s[nh][e], s[nh][2 + e]);
          m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
          m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
          m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
          mx[nh][e] = m;
          grew |= m > m_run[nh][e];
        }
      }
      if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
        for (int nh = 0; nh < NH; ++nh)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float m_new = fmaxf(m_run[nh][e], mx[nh][e]);
            const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_run[nh][e] - m_new);
            m_run[nh][e] = m_new;
            l_run[nh][e] *= alpha;
#pragma unroll
            for (int i = 0; i < NOT; ++i) { o[nh][i][e] *= alpha; o[nh][i][2 + e] *= alpha; }
          }
      }
      uint32_t pb[NH][2];   // P^T as B fragments: b0 = tokens 2j,2j+1 of head r, b1 = tokens 2j+8,2j+9
#pragma unroll
      for (int nh = 0; nh < NH; ++nh) {
        float pe[4];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float m_use = m_run[nh][e] == -INFINITY ? 0.f : m_run[nh][e];
          pe[e] = fast_exp2(s[nh][e] - m_use);
          pe[2 + e] = fast_exp2(s[nh][2 + e] - m_use);
          l_run[nh][e] += pe[e] + pe[2 + e];
        }
        pb[nh][0] = movmatrix_trans(pack_half2(pe[0] * vsc[0], pe[1] * vsc[0]));
        pb[nh][1] = movmatrix_trans(pack_half2(pe[2] * vsc[1], pe[3] * vsc[1]));
      }

      // ---- O^T += V^T P^T: rows = head-dims, k = the 16 tokens, columns = heads ---------------------------
      auto v_side = [&](auto patch_) {
        constexpr bool PATCH = decltype(patch_)::value;
        static_for<0, NVG>([&](auto g_) {
          constexpr int g = decltype(g_)::value;
          uint32_t lo[4], hi[4];
          static_for<0, 4>([&](auto i_) {
            constexpr int i = decltype(i_)::value;
            uint32_t idx; __half2 rr;
            ld.template vfield<i, g>(cur, idx, rr);
            const uint2 cw = *reinterpret_cast<const uint2*>(tblV + (idx * rstride + lane_off));
            lo[i] = hmul2_u32(cw.x, rr);
            hi[i] = hmul2_u32(cw.y, rr);
            if constexpr (PATCH) {
              const int c = r * NVG + g;
              if (c < N && ((vfl[i] >> c) & 1u)) {
                const uint32_t rel = vpre[i] + __popc(vfl[i] & ((1u << c) - 1u));
                ov_.load(ocur.offv + rel, rel, vinv[i], lo[i], hi[i]);
              }
            }
          });
          // tile 2g: rows r / r+8 = elements 0 / 1 of the lane's chunk; tile 2g+1: elements 2 / 3
          const uint32_t a0 = __byte_perm(lo[0], lo[1], 0x5410), a1 = __byte_perm(lo[0], lo[1], 0x7632);
          const uint32_t a2 = __byte_perm(lo[2], lo[3], 0x5410), a3 = __byte_perm(lo[2], lo[3], 0x7632);
          const uint32_t c0 = __byte_perm(hi[0], hi[1], 0x5410), c1 = __byte_perm(hi[0], hi[1], 0x7632);
          const uint32_t c2 = __byte_perm(hi[2], hi[3], 0x5410), c3 = __byte_perm(hi[2], hi[3], 0x7632);
#pragma unroll
          for (int nh = 0; nh < NH; ++nh) {
            mma16816(o[nh][2 * g], a0, a1, a2, a3, pb[nh][0], pb[nh][1]);
            mma16816(o[nh][2 * g + 1], c0, c1, c2, c3, pb[nh][0], pb[nh][1]);
          }
        });
      };
      if (OUTL && anyV) v_side(std::true_type{});
      else v_side(std::false_type{});
    };

    // ---- the warp's tiles, two at a time so that the prefetch buffers swap roles without copies ---------
    {
      typename Loader::Raw rawA, rawB;
      OutlRaw oA, oB;
      int tile = my_lo + warp;
      if (tile < my_hi) {
        if constexpr (OUTL) fetch_off(tile, offk_nn, offk_nn1, offv_nn, offv_nn1);
        fetch(rawA, oA, tile);
      }
      while (tile < my_hi) {
        if (tile + NW < my_hi) fetch(rawB, oB, tile + NW);
        compute(rawA, oA, tile);
        tile += NW;
        if (tile >= my_hi) break;
        if (tile + NW < my_hi) fetch(rawA, oA, tile + NW);
        compute(rawB, oB, tile);
        tile += NW;
      }
    }

    // ---- per-warp partial: o[d], m, l for every query head of this KV head -----------------------------
    const int n_parts = p.P * NW;
#pragma unroll
    for (int nh = 0; nh < NH; ++nh)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float l = l_run[nh][e];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        const int g = 8 * nh + 2 * j + e;
        if (g >= p.G) continue;
        const int64_t row = ((int64_t)b * p.Hq + h * p.G + g) * p.Tq + tq;
        float* dst = p.partials + (row * n_parts + part) * (p.d + 2);
#pragma unroll
        for (int i = 0; i < NOT; ++i) {
          const int chunk = r * NVG + (i >> 1);
          if (chunk < N) {
            dst[4 * chunk + 2 * (i & 1)] = o[nh][i][e];          // row r
            dst[4 * chunk + 2 * (i & 1) + 1] = o[nh][i][2 + e];  // row r+8
          }
        }
        if (r == 0) { dst[p.d] = m_run[nh][e]; dst[p.d + 1] = l; }
      }
  }
}

}  // namespace attn
}  // namespace hqmq
