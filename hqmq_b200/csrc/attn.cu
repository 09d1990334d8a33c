// Fused decode attention over the compressed KV cache (sm_100a).
//
// One CTA = (KV-range split, KV head, batch x query position); all G = H_q/H_kv query heads
// of the KV head share every decoded key/value.  Each warp walks 16-token tiles of its CTA's
// key range:
//   K side  codeword gather from the shared-memory table straight into mma.sync B fragments
//           (the head dimension is permuted so that one gathered 4-element codeword fills one
//           lane's two B registers), scaled by the integer radius code; S = Q K^T on tensor
//           cores (m16n8k16, fp16 in, fp32 accumulate); the per-token scale rs/qmax and the
//           softmax scale are applied to the fp32 scores.
//   softmax online (running max / sum per query head, exp2 domain).
//   V side  gather + radius, byte-permute token pairs into B fragments, O += P V on tensor
//           cores, the per-token V scale folded into P.
// Every warp writes an un-normalised partial (o[d], m, l) per query head; a second kernel
// merges the partials (and is also what merges partials gathered from other GPUs).
#include <math.h>
#include <string.h>

#include <type_traits>

#include "common.cuh"

namespace hqmq {
namespace {

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kTile = 16;

struct AttnParams {
  int B, Hq, Hkv, G, Tq, Tkv, d;
  int causal, window;
  float sscale;  // softmax_scale * log2(e) / qmax
  float vscale;  // 1 / qmax
  int n_splits, tiles_per_split;
  const void* Q; int q_dtype; int64_t qs_b, qs_h, qs_t;
  float* partials;  // [rows][n_parts][d+2]
  int n_parts;
  int layout;       // 0 native, 1 reference tuple
  int ib;           // index bits of a field (native: idx_bits; reference: 16)
  int table_rows;   // codewords per head in the shared-memory tables
  hqmq_packed K, V;
  const uint16_t* tblK; const uint16_t* tblV;
  hqmq_ref_packed Kr, Vr;
  const void* jK; const void* jV; int j_dtype;
};

__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, __half2 r) {
  __half2 v = __hmul2(*reinterpret_cast<__half2*>(&a), r);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Integer radius code (< 1024) as half2 (r, r): 0x6400 | r is the half 1024 + r.
__device__ __forceinline__ __half2 radius_half2(uint32_t rq) {
  uint32_t bits = 0x64006400u | rq | (rq << 16);
  return __hsub2(*reinterpret_cast<__half2*>(&bits), __float2half2_rn(1024.f));
}

template <int N>
struct Geo {
  static constexpr int NKS = N / 4;        // 16-wide k slices of the head dimension
  static constexpr int NVG = (N + 7) / 8;  // chunks per lane row on the V side
  static constexpr int NOT = NVG * 4;      // 8-wide output tiles (padded)
};

// Words a lane must read to cover `L` bits starting at bit j*L (j = 0..3) of a row.
constexpr int span_words(int L, int lanes) {
  int m = 0;
  for (int j = 0; j < lanes; ++j) {
    int w = (((j * L) & 31) + L + 31) / 32;
    if (w > m) m = w;
  }
  return m;
}

// ---- loaders ---------------------------------------------------------------------------------
// Raw data of one 16-token tile for one lane.  Lane (j = lane & 3, r = lane >> 2):
//   K side: tokens nt*8 + r (nt = 0,1), chunks j*NKS .. j*NKS + NKS-1
//   V side: tokens {2j, 2j+1, 2j+8, 2j+9}, chunks r*NVG .. r*NVG + NVG-1
//   scales of tokens {2j, 2j+1, 2j+8, 2j+9} for K and for V.

// Native layout, compile-time field width: rows are read as raw words and fields cut in registers.
template <int N, int CB>
struct FastLoader {
  static constexpr int NKS = Geo<N>::NKS, NVG = Geo<N>::NVG;
  static constexpr int LK = NKS * CB, LV = NVG * CB;
  static constexpr int KW = span_words(LK, 4), VW = span_words(LV, 8);
  struct Raw { uint32_t kw[2][KW + 1]; uint32_t vw[4][VW + 1]; uint32_t rsk[2], rsv[2]; };
  const uint8_t* kc; const uint8_t* vc; const uint16_t* krs; const uint16_t* vrs;
  int row_bytes, row_words, j, r, sdt;
  uint32_t idx_mask; int ib;

  __device__ FastLoader(const AttnParams& p, int b, int h, int lane) {
    const int64_t bh = (int64_t)b * p.Hkv + h;
    row_bytes = p.K.row_bytes; row_words = row_bytes >> 2;
    kc = p.K.codes + bh * p.K.T_cap * row_bytes;
    vc = p.V.codes + bh * p.V.T_cap * row_bytes;
    krs = reinterpret_cast<const uint16_t*>(p.K.rs) + bh * p.K.T_cap;
    vrs = reinterpret_cast<const uint16_t*>(p.V.rs) + bh * p.V.T_cap;
    j = lane & 3; r = lane >> 2; sdt = p.K.scale_dtype;
    ib = p.ib; idx_mask = (1u << ib) - 1u;
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
      const int t = t0 + nt * 8 + 2 * j;
      raw.rsk[nt] = *reinterpret_cast<const uint32_t*>(krs + t);
      raw.rsv[nt] = *reinterpret_cast<const uint32_t*>(vrs + t);
    }
  }
  template <int F>
  static __device__ __forceinline__ uint32_t cut(const uint32_t* w) {
    constexpr int bit = F * CB, a = bit >> 5, s = bit & 31;
    uint32_t v = (s + CB > 32) ? __funnelshift_r(w[a], w[a + 1], s) : (w[a] >> s);
    return v & ((1u << CB) - 1u);
  }
  template <int NT, int KS> __device__ __forceinline__ uint32_t kfield(const Raw& raw) const { return cut<KS>(raw.kw[NT]); }
  template <int I, int GG> __device__ __forceinline__ uint32_t vfield(const Raw& raw) const {
    uint32_t f = cut<GG>(raw.vw[I]);
    if constexpr (N % 8 != 0) { if (r * NVG + GG >= N) f = 0; }
    return f;
  }
  __device__ __forceinline__ float scale(uint32_t pair, int which) const {
    return bits16_to_float((uint16_t)(which ? (pair >> 16) : (pair & 0xffff)), sdt);
  }
  __device__ __forceinline__ float kscale(const Raw& raw, int nt, int e) const { return scale(raw.rsk[nt], e); }
  __device__ __forceinline__ float vscale(const Raw& raw, int nt, int e) const { return scale(raw.rsv[nt], e); }
};

// Any field width, native or reference layout: fields are extracted one by one at load time.
template <int N>
struct SlowLoader {
  static constexpr int NKS = Geo<N>::NKS, NVG = Geo<N>::NVG;
  struct Raw { uint32_t kf[2][NKS]; uint32_t vf[4][NVG]; float rsk[2][2], rsv[2][2]; };
  const AttnParams& p; int b, h, j, r;
  __device__ SlowLoader(const AttnParams& p_, int b_, int h_, int lane) : p(p_), b(b_), h(h_), j(lane & 3), r(lane >> 2) {}

  __device__ __forceinline__ uint32_t field(const hqmq_packed& pk, const hqmq_ref_packed& rf, int t, int c) const {
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
    if (p.layout == 0) {
      const int64_t row = ((int64_t)b * p.Hkv + h) * pk.T_cap + t;
      return load_scale(pk, row);
    }
    return load_float(rf.rs, b * rf.rs_stride[0] + h * rf.rs_stride[1] + t, rf.rs_dtype);
  }
  __device__ __forceinline__ void fetch(Raw& raw, int tile, int t_end) const {
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
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = t0 + nt * 8 + 2 * j + e;
        raw.rsk[nt][e] = t < t_end ? rscale(p.K, p.Kr, t) : 0.f;
        raw.rsv[nt][e] = t < t_end ? rscale(p.V, p.Vr, t) : 0.f;
      }
  }
  template <int NT, int KS> __device__ __forceinline__ uint32_t kfield(const Raw& raw) const { return raw.kf[NT][KS]; }
  template <int I, int GG> __device__ __forceinline__ uint32_t vfield(const Raw& raw) const { return raw.vf[I][GG]; }
  __device__ __forceinline__ float kscale(const Raw& raw, int nt, int e) const { return raw.rsk[nt][e]; }
  __device__ __forceinline__ float vscale(const Raw& raw, int nt, int e) const { return raw.rsv[nt][e]; }
};

template <int N, int CB> struct LoaderFor { using type = FastLoader<N, CB>; };
template <int N> struct LoaderFor<N, 0> { using type = SlowLoader<N>; };

// ---- compile-time unrolled helpers ----------------------------------------------------------------
template <int I, int End, class F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < End) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, End>(f);
  }
}

// ---- Med3x outliers ----------------------------------------------------------------------------------
// Flagged chunks keep their original 4 values in a side buffer.  They are merged by overwriting the
// decoded fragment with x * qmax / rs (the token's scale is its largest chunk norm, flagged chunks
// included, so the patched value never exceeds qmax in magnitude and cannot overflow fp16).
static_assert(kTile == HQMQ_OUT_BLOCK, "one outlier-offset entry per KV tile");

struct OutlRaw { uint32_t fk, fv, offk, offv; };   // lanes 0..15: flag words of the tile's tokens

struct OutlSide {
  const uint32_t* flags; const uint32_t* off; const unsigned char* vals; int dtype;
  __device__ __forceinline__ void init(const hqmq_packed& pk, int64_t bh) {
    flags = pk.flags ? pk.flags + bh * pk.T_cap : nullptr;
    off = pk.flags ? pk.out_off + bh * (pk.T_cap / HQMQ_OUT_BLOCK + 1) : nullptr;
    dtype = pk.out_dtype;
    vals = reinterpret_cast<const unsigned char*>(pk.out_vals) + bh * pk.out_cap * 4 * (dtype == HQMQ_F32 ? 4 : 2);
  }
  // original values of payload entry `pos`, scaled by `inv`, as two half2 registers
  __device__ __forceinline__ void load(uint32_t pos, float inv, uint32_t& lo, uint32_t& hi) const {
    float x0, x1, x2, x3;
    if (dtype == HQMQ_F32) {
      const float4 v = *reinterpret_cast<const float4*>(vals + (int64_t)pos * 16);
      x0 = v.x; x1 = v.y; x2 = v.z; x3 = v.w;
    } else {
      const uint2 v = *reinterpret_cast<const uint2*>(vals + (int64_t)pos * 8);
      x0 = bits16_to_float((uint16_t)(v.x & 0xffff), dtype); x1 = bits16_to_float((uint16_t)(v.x >> 16), dtype);
      x2 = bits16_to_float((uint16_t)(v.y & 0xffff), dtype); x3 = bits16_to_float((uint16_t)(v.y >> 16), dtype);
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

template <int N, int CB, bool OUTL>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const AttnParams p) {
  using G_ = Geo<N>;
  using Loader = typename LoaderFor<N, CB>::type;
  constexpr int NKS = G_::NKS, NVG = G_::NVG, NOT = G_::NOT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint2* tblK = reinterpret_cast<uint2*>(smem_raw);
  uint2* tblV = tblK + p.table_rows;

  const int split = blockIdx.x, h = blockIdx.y;
  const int b = blockIdx.z / p.Tq, tq = blockIdx.z - b * p.Tq;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = lane & 3, r = lane >> 2;

  // ---- codeword tables into shared memory (fp16 x 4 per entry) -----------------------------------
  if (p.layout == 0) {
    const uint2* gk = reinterpret_cast<const uint2*>(p.tblK) + (int64_t)h * p.table_rows;
    const uint2* gv = reinterpret_cast<const uint2*>(p.tblV) + (int64_t)h * p.table_rows;
    for (int i = threadIdx.x; i < p.table_rows; i += kAttnThreads) { tblK[i] = gk[i]; tblV[i] = gv[i]; }
  } else {
    for (int i = threadIdx.x; i < p.table_rows; i += kAttnThreads) {
      const int64_t base = ((int64_t)h * p.table_rows + i) * 4;
      float k0 = load_float(p.jK, base, p.j_dtype), k1 = load_float(p.jK, base + 1, p.j_dtype);
      float k2 = load_float(p.jK, base + 2, p.j_dtype), k3 = load_float(p.jK, base + 3, p.j_dtype);
      float v0 = load_float(p.jV, base, p.j_dtype), v1 = load_float(p.jV, base + 1, p.j_dtype);
      float v2 = load_float(p.jV, base + 2, p.j_dtype), v3 = load_float(p.jV, base + 3, p.j_dtype);
      tblK[i] = make_uint2(pack_half2(k0, k1), pack_half2(k2, k3));
      tblV[i] = make_uint2(pack_half2(v0, v1), pack_half2(v2, v3));
    }
  }
  __syncthreads();

  // ---- key range of this CTA ------------------------------------------------------------------------
  const int t_end = p.causal ? min(p.Tkv, tq + 1) : p.Tkv;
  const int t_beg = p.window > 0 ? max(0, t_end - p.window) : 0;
  const int tile_lo = t_beg / kTile, tile_hi = (t_end + kTile - 1) / kTile;
  const int my_lo = tile_lo + split * p.tiles_per_split;
  const int my_hi = min(tile_hi, my_lo + p.tiles_per_split);

  // ---- Q fragments: row r (and r+8) = query head, k slots {2j,2j+1,2j+8,2j+9} = one chunk ----------
  uint32_t qa[NKS][4];
  {
    const int64_t qb = (int64_t)b * p.qs_b + (int64_t)tq * p.qs_t;
#pragma unroll
    for (int ks = 0; ks < NKS; ++ks) {
      const int dim = 4 * (j * NKS + ks);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int g = r + 8 * hh;
        float q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
        if (g < p.G) {
          const int64_t o = qb + (int64_t)(h * p.G + g) * p.qs_h + dim;
          q0 = load_float(p.Q, o, p.q_dtype); q1 = load_float(p.Q, o + 1, p.q_dtype);
          q2 = load_float(p.Q, o + 2, p.q_dtype); q3 = load_float(p.Q, o + 3, p.q_dtype);
        }
        qa[ks][hh] = pack_half2(q0, q1);      // a0 (hh=0) / a1 (hh=1)
        qa[ks][2 + hh] = pack_half2(q2, q3);  // a2 / a3
      }
    }
  }

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[NOT][4];
#pragma unroll
  for (int i = 0; i < NOT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  Loader ld(p, b, h, lane);
  typename Loader::Raw cur, nxt;
  OutlSide ok_, ov_;
  OutlRaw ocur = {0, 0, 0, 0}, onxt = {0, 0, 0, 0};
  if constexpr (OUTL) {
    ok_.init(p.K, (int64_t)b * p.Hkv + h);
    ov_.init(p.V, (int64_t)b * p.Hkv + h);
  }
  auto fetch_outl = [&](OutlRaw& o, int tl) {
    o.fk = o.fv = o.offk = o.offv = 0;
    const int tt = tl * kTile + (lane & 15);
    if (lane < 16 && tt < t_end) {
      if (ok_.flags) o.fk = ok_.flags[tt];
      if (ov_.flags) o.fv = ov_.flags[tt];
    }
    if (ok_.flags) o.offk = ok_.off[tl];
    if (ov_.flags) o.offv = ov_.off[tl];
  };
  int tile = my_lo + warp;
  if (tile < my_hi) {
    ld.fetch(cur, tile, t_end);
    if constexpr (OUTL) fetch_outl(ocur, tile);
  }

  for (; tile < my_hi; tile += kAttnWarps) {
    const int tn = tile + kAttnWarps;
    if (tn < my_hi) {
      ld.fetch(nxt, tn, t_end);
      if constexpr (OUTL) fetch_outl(onxt, tn);
    }
    const int t0 = tile * kTile;

    // ---- outlier bookkeeping of this tile -------------------------------------------------------------
    bool anyK = false, anyV = false;
    uint32_t kfl[2] = {0, 0}, kpre[2] = {0, 0}, vfl[4] = {0, 0, 0, 0}, vpre[4] = {0, 0, 0, 0};
    float kinv[2] = {0.f, 0.f};
    if constexpr (OUTL) {
      anyK = __ballot_sync(0xffffffffu, ocur.fk != 0) != 0;
      anyV = __ballot_sync(0xffffffffu, ocur.fv != 0) != 0;
      if (anyK) {
        const uint32_t ex = excl_scan16(__popc(ocur.fk), lane) + ocur.offk;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          kfl[nt] = __shfl_sync(0xffffffffu, ocur.fk, nt * 8 + r);
          kpre[nt] = __shfl_sync(0xffffffffu, ex, nt * 8 + r);
          // the K-side lane owns token nt*8 + r; its scale is not among the ones the tile data carries
          const int t = t0 + nt * 8 + r;
          kinv[nt] = (kfl[nt] && t < t_end) ? (float)((1 << p.K.radius_bits) - 1) / load_scale(p.K, ((int64_t)b * p.Hkv + h) * p.K.T_cap + t) : 0.f;
        }
      }
      if (anyV) {
        const uint32_t ex = excl_scan16(__popc(ocur.fv), lane) + ocur.offv;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tl = 2 * j + (i & 1) + (i >> 1) * 8;
          vfl[i] = __shfl_sync(0xffffffffu, ocur.fv, tl);
          vpre[i] = __shfl_sync(0xffffffffu, ex, tl);
        }
      }
    }

    // ---- S = Q K^T ---------------------------------------------------------------------------------
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
    static_for<0, 2>([&](auto nt_) {
      constexpr int nt = decltype(nt_)::value;
      static_for<0, NKS>([&](auto ks_) {
        constexpr int ks = decltype(ks_)::value;
        const uint32_t f = ld.template kfield<nt, ks>(cur);
        const uint2 cw = tblK[f & ((1u << p.ib) - 1u)];
        const __half2 rr = radius_half2(f >> p.ib);
        uint32_t b0 = hmul2_u32(cw.x, rr), b1 = hmul2_u32(cw.y, rr);
        if constexpr (OUTL) {
          if (anyK) {
            const int c = j * NKS + ks;
            if ((kfl[nt] >> c) & 1u) ok_.load(kpre[nt] + __popc(kfl[nt] & ((1u << c) - 1u)), kinv[nt], b0, b1);
          }
        }
        mma16816(s[nt], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
      });
    });

    // ---- scale, mask, online softmax -------------------------------------------------------------------
    float pv[2][4];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = t0 + nt * 8 + 2 * j + e;
        const bool ok = t >= t_beg && t < t_end;
        const float sc = ld.kscale(cur, nt, e) * p.sscale;
        s[nt][e] = ok ? s[nt][e] * sc : -INFINITY;
        s[nt][2 + e] = ok ? s[nt][2 + e] * sc : -INFINITY;
        mx[0] = fmaxf(mx[0], s[nt][e]);
        mx[1] = fmaxf(mx[1], s[nt][2 + e]);
      }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
      mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const float m_new = fmaxf(m_run[hh], mx[hh]);
      m_use[hh] = m_new == -INFINITY ? 0.f : m_new;
      alpha[hh] = exp2f(m_run[hh] - m_use[hh]);
      m_run[hh] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float p0 = exp2f(s[nt][e] - m_use[0]);
        const float p1 = exp2f(s[nt][2 + e] - m_use[1]);
        psum[0] += p0; psum[1] += p1;
        const int t = t0 + nt * 8 + 2 * j + e;
        const float vs = (t >= t_beg && t < t_end) ? ld.vscale(cur, nt, e) * p.vscale : 0.f;
        pv[nt][e] = p0 * vs;
        pv[nt][2 + e] = p1 * vs;
      }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) l_run[hh] = l_run[hh] * alpha[hh] + psum[hh];
#pragma unroll
    for (int i = 0; i < NOT; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }

    // ---- O += P V -----------------------------------------------------------------------------------------
    const uint32_t pa0 = pack_half2(pv[0][0], pv[0][1]), pa1 = pack_half2(pv[0][2], pv[0][3]);
    const uint32_t pa2 = pack_half2(pv[1][0], pv[1][1]), pa3 = pack_half2(pv[1][2], pv[1][3]);
    static_for<0, NVG>([&](auto g_) {
      constexpr int g = decltype(g_)::value;
      uint32_t lo[4], hi[4];
      static_for<0, 4>([&](auto i_) {
        constexpr int i = decltype(i_)::value;
        const uint32_t f = ld.template vfield<i, g>(cur);
        const uint2 cw = tblV[f & ((1u << p.ib) - 1u)];
        const __half2 rr = radius_half2(f >> p.ib);
        lo[i] = hmul2_u32(cw.x, rr);
        hi[i] = hmul2_u32(cw.y, rr);
        if constexpr (OUTL) {
          if (anyV) {
            const int c = r * NVG + g;
            if (c < N && ((vfl[i] >> c) & 1u)) {
              const float rsv = ld.vscale(cur, i >> 1, i & 1);
              ov_.load(vpre[i] + __popc(vfl[i] & ((1u << c) - 1u)), (float)((1 << p.V.radius_bits) - 1) / rsv, lo[i], hi[i]);
            }
          }
        }
      });
      mma16816(o[g * 4 + 0], pa0, pa1, pa2, pa3, __byte_perm(lo[0], lo[1], 0x5410), __byte_perm(lo[2], lo[3], 0x5410));
      mma16816(o[g * 4 + 1], pa0, pa1, pa2, pa3, __byte_perm(lo[0], lo[1], 0x7632), __byte_perm(lo[2], lo[3], 0x7632));
      mma16816(o[g * 4 + 2], pa0, pa1, pa2, pa3, __byte_perm(hi[0], hi[1], 0x5410), __byte_perm(hi[2], hi[3], 0x5410));
      mma16816(o[g * 4 + 3], pa0, pa1, pa2, pa3, __byte_perm(hi[0], hi[1], 0x7632), __byte_perm(hi[2], hi[3], 0x7632));
    });
    cur = nxt;
    if constexpr (OUTL) ocur = onxt;
  }

  // ---- per-warp partial: o[d], m, l for every query head of this KV head ---------------------------
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
    l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
  }
  const int part = split * kAttnWarps + warp;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int g = r + 8 * hh;
    if (g >= p.G) continue;
    const int64_t row = ((int64_t)b * p.Hq + h * p.G + g) * p.Tq + tq;
    float* dst = p.partials + (row * p.n_parts + part) * (p.d + 2);
#pragma unroll
    for (int i = 0; i < NOT; ++i) {
      const int gi = i >> 2, e = i & 3;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int chunk = (2 * j + cc) * NVG + gi;
        if (chunk < N) dst[4 * chunk + e] = o[i][2 * hh + cc];
      }
    }
    if (j == 0) { dst[p.d] = m_run[hh]; dst[p.d + 1] = l_run[hh]; }
  }
}

// Merge partials: parts [rows][n_parts][d+2] -> normalised output rows (or one merged partial).
__global__ void combine_kernel(const float* __restrict__ parts, int n_parts, int64_t rows, int d, int out_dtype,
                               void* __restrict__ out, int64_t out_row_stride_b, int64_t os_b, int64_t os_h, int64_t os_t,
                               int Hq, int Tq, float* __restrict__ merged) {
  const int64_t row = blockIdx.x;
  if (row >= rows) return;
  const float* base = parts + row * n_parts * (d + 2);
  float m_star = -INFINITY;
  for (int i = 0; i < n_parts; ++i) m_star = fmaxf(m_star, base[i * (d + 2) + d]);
  const float m_use = m_star == -INFINITY ? 0.f : m_star;
  float l_star = 0.f;
  for (int i = 0; i < n_parts; ++i) l_star += base[i * (d + 2) + d + 1] * exp2f(base[i * (d + 2) + d] - m_use);
  for (int x = threadIdx.x; x < d; x += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < n_parts; ++i) {
      const float w = exp2f(base[i * (d + 2) + d] - m_use);
      if (w != 0.f) acc += base[i * (d + 2) + x] * w;
    }
    if (merged) {
      merged[row * (d + 2) + x] = acc;
    } else {
      const float v = l_star > 0.f ? acc / l_star : 0.f;
      // row = (b*Hq + hq)*Tq + tq
      const int64_t tq = row % Tq, bh = row / Tq, hq = bh % Hq, b = bh / Hq;
      store_float(out, b * os_b + hq * os_h + tq * os_t + x, v, out_dtype);
    }
  }
  if (merged && threadIdx.x == 0) { merged[row * (d + 2) + d] = m_star; merged[row * (d + 2) + d + 1] = l_star; }
}

struct Plan { int n_splits, tiles_per_split, n_parts; size_t ws_bytes; int table_rows; size_t smem; };

int make_plan(const hqmq_attn_args* a, Plan& pl) {
  const int max_keys = a->T_kv;
  const int keys = a->window > 0 ? (a->window < max_keys ? a->window : max_keys) : max_keys;
  int tiles = (keys + kTile - 1) / kTile + 1;  // +1: a window may straddle one more tile
  if (tiles < 1) tiles = 1;
  int splits = a->kv_splits;
  const int64_t units = (int64_t)a->B * a->H_kv * a->T_q;
  if (splits <= 0) {
    const int64_t target = 148 * 4;
    splits = (int)((target + units - 1) / units);
    const int max_splits = (tiles + 2 * kAttnWarps - 1) / (2 * kAttnWarps);
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
  }
  if (splits > tiles) splits = tiles;
  pl.n_splits = splits;
  pl.tiles_per_split = (tiles + splits - 1) / splits;
  pl.n_parts = splits * kAttnWarps;
  const int64_t rows = (int64_t)a->B * a->H_q * a->T_q;
  pl.ws_bytes = (size_t)rows * pl.n_parts * (a->d + 2) * sizeof(float);
  pl.table_rows = a->layout == 0 ? 24 * a->K.S : a->K_size;
  pl.smem = (size_t)pl.table_rows * 8 * 2;
  return HQMQ_OK;
}

int validate_attn(const hqmq_attn_args* a) {
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

template <int N, int CB, bool OUTL>
int launch(const AttnParams& p, const Plan& pl, cudaStream_t st) {
  auto kern = attn_decode_kernel<N, CB, OUTL>;
  if (pl.smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) != cudaSuccess)
      return HQMQ_ERR_CUDA;
  }
  dim3 grid(pl.n_splits, p.Hkv, p.B * p.Tq);
  kern<<<grid, kAttnThreads, pl.smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? HQMQ_OK : HQMQ_ERR_CUDA;
}

template <int N, bool OUTL>
int dispatch_cb(const AttnParams& p, const Plan& pl, int cb, bool fast_ok, cudaStream_t st) {
  if constexpr (N == 16 || N == 32) {
    if (fast_ok) {
      if (cb == 13) return launch<N, 13, OUTL>(p, pl, st);
      if (cb == 16) return launch<N, 16, OUTL>(p, pl, st);
      if (cb == 19) return launch<N, 19, OUTL>(p, pl, st);
    }
  }
  return launch<N, 0, OUTL>(p, pl, st);
}
template <int N>
int dispatch_outl(const AttnParams& p, const Plan& pl, int cb, bool fast_ok, bool outl, cudaStream_t st) {
  return outl ? dispatch_cb<N, true>(p, pl, cb, fast_ok, st) : dispatch_cb<N, false>(p, pl, cb, fast_ok, st);
}

}  // namespace
}  // namespace hqmq

using namespace hqmq;

extern "C" size_t hqmq_attn_workspace_bytes(const hqmq_attn_args* a) {
  if (validate_attn(a) != HQMQ_OK) return 0;
  Plan pl;
  make_plan(a, pl);
  return pl.ws_bytes;
}

extern "C" int hqmq_combine_partials(const float* parts, int n_parts, int64_t rows, int d, int out_dtype, void* out,
                                     void* stream) {
  if (!parts || !out) return HQMQ_ERR_ARG;
  if (n_parts < 1 || rows < 0 || d < 1) return HQMQ_ERR_SHAPE;
  if (!is_float_dtype(out_dtype)) return HQMQ_ERR_DTYPE;
  if (rows == 0) return HQMQ_OK;
  // rows are laid out contiguously: treat as B = rows, Hq = Tq = 1
  combine_kernel<<<(unsigned)rows, 128, 0, (cudaStream_t)stream>>>(parts, n_parts, rows, d, out_dtype, out, 0, d, 0, 0, 1, 1,
                                                                  nullptr);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

extern "C" int hqmq_attn_decode(const hqmq_attn_args* a, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = validate_attn(a);
  if (rc) return rc;
  Plan pl;
  make_plan(a, pl);
  if (!workspace || workspace_bytes < pl.ws_bytes) return HQMQ_ERR_WORKSPACE;
  if ((uintptr_t)workspace & 15) return HQMQ_ERR_ALIGN;
  if (pl.smem > 220 * 1024) return HQMQ_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;

  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.B = a->B; p.Hq = a->H_q; p.Hkv = a->H_kv; p.G = a->H_q / a->H_kv; p.Tq = a->T_q; p.Tkv = a->T_kv; p.d = a->d;
  p.causal = a->causal; p.window = a->window;
  const float scale = a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / sqrtf((float)a->d);
  p.sscale = scale * 1.4426950408889634f / (float)a->r_qmax;
  p.vscale = 1.0f / (float)a->r_qmax;
  p.n_splits = pl.n_splits; p.tiles_per_split = pl.tiles_per_split; p.n_parts = pl.n_parts;
  p.Q = a->Q; p.q_dtype = a->q_dtype; p.qs_b = a->q_stride[0]; p.qs_h = a->q_stride[1]; p.qs_t = a->q_stride[2];
  p.partials = reinterpret_cast<float*>(workspace);
  p.layout = a->layout;
  p.table_rows = pl.table_rows;
  const int n = a->d / 4;
  int cb = 0;
  bool fast_ok = false;
  if (a->layout == 0) {
    p.K = a->K; p.V = a->V; p.tblK = a->table_K; p.tblV = a->table_V;
    p.ib = idx_bits_for(a->K.S);
    cb = p.ib + a->K.radius_bits;
    fast_ok = is_half_dtype(a->K.scale_dtype) && a->K.row_bytes == n * cb / 8 && (n * cb) % 32 == 0;
  } else {
    p.Kr = a->K_ref; p.Vr = a->V_ref; p.jK = a->joint_K; p.jV = a->joint_V; p.j_dtype = a->joint_dtype;
    p.ib = 16;
  }
  const bool outl = a->layout == 0 && (a->K.flags != nullptr || a->V.flags != nullptr);
  switch (n) {
    case 4: rc = dispatch_outl<4>(p, pl, cb, fast_ok, outl, st); break;
    case 8: rc = dispatch_outl<8>(p, pl, cb, fast_ok, outl, st); break;
    case 12: rc = dispatch_outl<12>(p, pl, cb, fast_ok, outl, st); break;
    case 16: rc = dispatch_outl<16>(p, pl, cb, fast_ok, outl, st); break;
    case 32: rc = dispatch_outl<32>(p, pl, cb, fast_ok, outl, st); break;
    default: return HQMQ_ERR_UNSUPPORTED;
  }
  if (rc) return rc;
  const int64_t rows = (int64_t)a->B * a->H_q * a->T_q;
  combine_kernel<<<(unsigned)rows, a->d < 128 ? 64 : 128, 0, st>>>(
      p.partials, pl.n_parts, rows, a->d, a->o_dtype, a->O, 0, a->o_stride[0], a->o_stride[1], a->o_stride[2], a->H_q,
      a->T_q, a->partials_only ? a->partials : nullptr);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}
