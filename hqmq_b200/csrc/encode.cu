// KV-cache encoder for sm_100a: chunk norms, per-token-max radius codes, nearest codeword of
// the 24*S product codebook, Med3x median / flags / outlier side buffer, bit-packed rows.
//
// Arithmetic contract (bit-exact with the reference evaluated on the fp32 upcast of x):
//   norm   = sqrt(((x0^2 + x1^2) + x2^2) + x3^2), every op a separate IEEE fp32 op
//   radius = max(norm, 1e-8); r_max = max over the token's chunks (flagged ones included)
//   rq     = clamp(rint((radius / (r_max / qmax))), 0, qmax) with two IEEE divisions
//   idx    = argmax_k <x/radius, joint[k]>; exhaustive search evaluates, for every secondary
//            s, y = u * conj(q_s) and snaps y to the 24-cell in closed form
//   med    = torch.quantile(norms of the head, 0.5): the two middle order statistics a <= b,
//            med = a if N odd else b - (b - a) * 0.5; flag = norm > med * C (strict)
// A flagged chunk keeps its index but its stored radius code is 0: its values live in the side buffer.
#include <string.h>

#include "common.cuh"

namespace hqmq {

namespace {

constexpr int kEncThreads = 512;
constexpr int kEncWarps = kEncThreads / 32;
constexpr int kEncIters = 8;      // token groups per block
constexpr int kHistBins = 2048;   // 11-bit digits: bits [31:21], [20:10], then 10 bits [9:0]
constexpr int kMaxRowWords = 20;
constexpr int kBandWords = 4;     // per head: thr_lo bits, thr_hi bits, undecided chunks seen, spare
constexpr int kUndCap = 4096;     // undecided chunks listed per head; more -> the fix-up re-scans x instead

// ---- nearest-codeword look-up table -------------------------------------------------------------------
// The joint codebook {p * q_s} is invariant under left multiplication by any of the 24 Hurwitz units g, so the
// unit direction u is first FOLDED by its nearest unit: v = conj(g) * u lies in the Voronoi cell of 1 among the 24
// units, which in the coordinates w = (v1, v2, v3) / v0 is the octahedron |w1| + |w2| + |w3| <= 1, and the nearest
// codeword of u is g times the nearest codeword of v (a 24 x 24 index table).  (Folding by the nearest unit is
// closed form: the larger of the largest |u_i| and (|u0|+|u1|+|u2|+|u3|)/2 names it; conj(g) * u is a signed
// permutation for an axis unit and sums of differences of the |u_i| for a half-integer unit.)
// A grid of n cells per axis covers the octahedron (only the cells that meet it are stored: a row table over
// (cx, cy) gives the first stored cz and where the row's cells start).  Each cell names every codeword that can be
// the nearest one for some direction in the (slightly grown) cell: all k not beaten over the whole cell by the
// winner at the cell's centre, minus those beaten over the whole cell by another listed one -- the comparison of
// two codewords is linear in w, so its extreme over the box is at a corner.  A cell with ONE possible winner stores
// it in its own word (no similarity is evaluated at all); the others point at a list, padded to groups of four,
// which is evaluated with the same fp32 dot product an exhaustive scan of the joint table would use.  At n = 48
// and S = 96 a list holds 1.9 codewords on average (8 at most) and 98 % of the lists are one group.
constexpr int kLutNMax = 48;
constexpr int kLutRows = kLutNMax * kLutNMax;
constexpr int kLutCellCap = 24576;          // stored cells (23.4 k at n = 48)
constexpr int kLutCandCap = 65532;          // candidate entries per head (list offsets / 4 are 15-bit cell words)
constexpr int kLutMaxList = 16;             // longest list a cell may have; longer -> exhaustive search there
constexpr float kLutBoxEps = 1e-5f;         // the boxes are grown by this much (cell assignment rounding)
constexpr float kLutMargin = 1e-5f;         // a codeword is dropped only if it loses by more than this
// device layout of a table (bytes): global header {n, n_cells, ...} | rows[kLutRows] uint32 = base (20 bits) |
// first stored cz (6) | stored cells of the row (6) | per head: {total candidates, valid, -, -} uint32, then
// cells[kLutCellCap] uint16 (0xFFFF: exhaustive; bit 15: the single winner in bits 0..14; else list offset / 4),
// cands[kLutCandCap] uint16 (bit 15 of a group's first entry marks the list's last group)
constexpr size_t kLutOffRows = 32;
constexpr size_t kLutOffHeads = kLutOffRows + (size_t)kLutRows * 4;
constexpr size_t kLutHeadBytes = 16 + (size_t)kLutCellCap * 2 + (size_t)kLutCandCap * 2;

struct Mul24 { uint8_t v[24][24]; };       // reference index of (unit g) * (primary p)

struct Maps24 { uint8_t ref_to_native[24]; };

struct EncGeom {
  int B, H, T_new, n, npl, tpw;  // npl = lanes per token (power of two >= n), tpw = tokens per warp
  int S, ib, rbits, qmax;
  int x_dtype;
  int64_t xs_b, xs_h, xs_t;
  // d_head 64 through the kernels written for 32 chunks per token: with the tokens contiguous in memory, an even
  // token count and an even first row, two consecutive tokens form one "token" of 32 chunks (T_new, xs_t and the
  // packed rows are then those of the pairs); what is per token -- the maximum radius, the scale, the flag word, the
  // row number -- is taken per half-warp.
  int pair16;
};

// Workspace layout (uint32 words)
struct EncWs {
  uint32_t* status;   // [4]
  uint32_t* hist;     // [H][3 levels][2 queries][kHistBins]
  uint32_t* sel;      // [H][8]: prefix_lo, rank_lo, prefix_hi, rank_hi, a_bits, b_bits, thr_bits, med_bits
};

__device__ __forceinline__ void load_chunk(const void* x, int64_t off, int dtype, float v[4]) {
  if (dtype == HQMQ_F32) {
    float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + off);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
  } else {
    uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(x) + off);
    uint16_t a = r.x & 0xffff, b = r.x >> 16, c = r.y & 0xffff, d = r.y >> 16;
    v[0] = bits16_to_float(a, dtype); v[1] = bits16_to_float(b, dtype);
    v[2] = bits16_to_float(c, dtype); v[3] = bits16_to_float(d, dtype);
  }
}

__device__ __forceinline__ float chunk_norm(const float v[4]) {
  float s = __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(v[0], v[0]), __fmul_rn(v[1], v[1])), __fmul_rn(v[2], v[2])),
                      __fmul_rn(v[3], v[3]));
  return __fsqrt_rn(s);
}

// Closed-form nearest 24-cell vertex to y: returns similarity and writes the reference
// primary index (axis candidates 0..7, half-integer candidates 8..23).
__device__ __forceinline__ float snap24(float y0, float y1, float y2, float y3, int& p) {
  float a0 = fabsf(y0), a1 = fabsf(y1), a2 = fabsf(y2), a3 = fabsf(y3);
  float best = a0; int ax = 0;
  if (a1 > best) { best = a1; ax = 1; }
  if (a2 > best) { best = a2; ax = 2; }
  if (a3 > best) { best = a3; ax = 3; }
  float yv = ax == 0 ? y0 : ax == 1 ? y1 : ax == 2 ? y2 : y3;
  p = 2 * ax + (yv < 0.f ? 1 : 0);
  float half = 0.5f * (((a0 + a1) + a2) + a3);
  if (half > best) {
    best = half;
    p = 8 + ((y0 < 0.f) << 3) + ((y1 < 0.f) << 2) + ((y2 < 0.f) << 1) + (y3 < 0.f);
  }
  return best;
}

// Exhaustive search: for every secondary quaternion q_s (shared memory, fp32), rotate the
// unit direction by conj(q_s) and snap.  Ties keep the smallest reference index p*S + s.
__device__ __forceinline__ int search_exhaustive(const float4* __restrict__ qs, int S, float u0, float u1, float u2,
                                                 float u3, int& best_s) {
  float best = -1.f; int bp = 0, bs = 0;
  for (int s = 0; s < S; ++s) {
    float4 q = qs[s];
    float y0 = u0 * q.x + u1 * q.y + u2 * q.z + u3 * q.w;
    float y1 = -u0 * q.y + u1 * q.x - u2 * q.w + u3 * q.z;
    float y2 = -u0 * q.z + u1 * q.w + u2 * q.x - u3 * q.y;
    float y3 = -u0 * q.w - u1 * q.z + u2 * q.y + u3 * q.x;
    int p;
    float sim = snap24(y0, y1, y2, y3, p);
    if (sim > best || (sim == best && p < bp)) { best = sim; bp = p; bs = s; }
  }
  best_s = bs;
  return bp;
}

// A table as a kernel sees it (global or shared memory).
struct LutView {
  const uint32_t* rows; const uint16_t* cells; const uint16_t* cands;
  const uint8_t* nm;     // [24][24]: (fold unit g, primary p of the folded winner) -> primary of g * p, in the form the caller wants
  int n; float hn;       // cells per axis, n / 2
};

__device__ __forceinline__ float xor_sign(float x, uint32_t sign_bits) { return __uint_as_float(__float_as_uint(x) ^ sign_bits); }
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The order statistics torch.quantile(flat, q) interpolates between and its weight, with torch's own arithmetic
// (ATen quantile_compute: rank = fl32(fl32(q) * fl32(N - 1)), below = trunc, above = ceil, weight = rank - below;
// lerp with one fused multiply-add, a + w * (b - a) for w < 0.5, else b - (b - a) * (1 - w)).  q <= 0 names the
// median of Med3x with exact integer ranks: (N - 1) / 2 and N / 2, weight 0.5 for an even count.
struct QRank { uint64_t lo, hi; float w; };
__host__ __device__ inline QRank quantile_rank(uint64_t N, float q) {
  QRank r;
  if (!(q > 0.f)) { r.lo = (N - 1) / 2; r.hi = N / 2; r.w = (N & 1) ? 0.f : 0.5f; return r; }
  volatile float last = (float)(N - 1);
  volatile float rf = q * last;
  const float rfl = rf;
  r.lo = (uint64_t)rfl;
  r.hi = (uint64_t)ceilf(rfl);
  r.w = rfl - (float)r.lo;
  return r;
}
__device__ __forceinline__ float quantile_lerp(float a, float b, float w) {
  const float diff = __fsub_rn(b, a);
  return w < 0.5f ? __fmaf_rn(w, diff, a) : __fmaf_rn(-diff, __fsub_rn(1.f, w), b);
}

// Nearest codeword of the direction u through the table: writes nm[g][p'] and the secondary index, returns
// false when the chunk has to take the exhaustive search (zero direction, a cell without a list).
__device__ __forceinline__ bool search_fold24(const float4* __restrict__ joint, const LutView& L, int S, float inv_S,
                                              float u0, float u1, float u2, float u3, int& prim, int& sidx) {
  const float a0 = fabsf(u0), a1 = fabsf(u1), a2 = fabsf(u2), a3 = fabsf(u3);
  int ax = 0; float am = a0;
  if (a1 > am) { am = a1; ax = 1; }
  if (a2 > am) { am = a2; ax = 2; }
  if (a3 > am) { am = a3; ax = 3; }
  if (!(am > 0.f)) return false;
  const float hs = ((a0 + a1) + a2) + a3;          // twice the similarity of the nearest half-integer unit
  int gp; float v0, v1, v2, v3;
  if (hs > 2.f * am) {
    // g = (s0, s1, s2, s3) / 2 with s_i = sign(u_i); 2 conj(g) u in terms of the |u_i|
    const uint32_t b0 = __float_as_uint(u0), b1 = __float_as_uint(u1), b2 = __float_as_uint(u2), b3 = __float_as_uint(u3);
    gp = 8 + (int)(((b0 >> 31) << 3) | ((b1 >> 31) << 2) | ((b2 >> 31) << 1) | (b3 >> 31));
    v0 = hs;
    v1 = xor_sign(a1 - a0, (b0 ^ b1) & 0x80000000u) + xor_sign(a2 - a3, (b2 ^ b3) & 0x80000000u);
    v2 = xor_sign(a2 - a0, (b0 ^ b2) & 0x80000000u) + xor_sign(a3 - a1, (b1 ^ b3) & 0x80000000u);
    v3 = xor_sign(a3 - a0, (b0 ^ b3) & 0x80000000u) + xor_sign(a1 - a2, (b1 ^ b2) & 0x80000000u);
  } else {
    if (ax == 0) { v0 = u0; v1 = u1; v2 = u2; v3 = u3; }
    else if (ax == 1) { v0 = u1; v1 = -u0; v2 = u3; v3 = -u2; }
    else if (ax == 2) { v0 = u2; v1 = -u3; v2 = -u0; v3 = u1; }
    else { v0 = u3; v1 = u2; v2 = -u1; v3 = -u0; }
    const bool neg = v0 < 0.f;
    if (neg) { v0 = -v0; v1 = -v1; v2 = -v2; v3 = -v3; }
    gp = 2 * ax + (neg ? 1 : 0);
  }
  const float inv = rcp_approx(v0) * L.hn;
  const int cx = min(L.n - 1, max(0, (int)fmaf(v1, inv, L.hn)));
  const int cy = min(L.n - 1, max(0, (int)fmaf(v2, inv, L.hn)));
  const int cz = (int)fmaf(v3, inv, L.hn);
  const uint32_t row = L.rows[cx * L.n + cy];
  const int zcnt = (int)(row >> 26);
  if (zcnt == 0) return false;
  const int zc = min(zcnt - 1, max(0, cz - (int)((row >> 20) & 63u)));
  const uint32_t cw = L.cells[(row & 0xfffffu) + zc];
  if (cw == 0xffffu) return false;
  int bk;
  if (cw & 0x8000u) {
    bk = (int)(cw & 0x7fffu);
  } else {
    float best = -3.f;
    bk = 0;
    const uint16_t* e = L.cands + cw * 4u;
    for (;;) {
      const uint2 kk = *reinterpret_cast<const uint2*>(e);
      const int k0 = kk.x & 0x7fff, k1 = kk.x >> 16, k2 = kk.y & 0xffff, k3 = kk.y >> 16;
      const float4 c0 = joint[k0], c1 = joint[k1], c2 = joint[k2], c3 = joint[k3];
      const float s0 = fmaf(v3, c0.w, fmaf(v2, c0.z, fmaf(v1, c0.y, v0 * c0.x)));
      const float s1 = fmaf(v3, c1.w, fmaf(v2, c1.z, fmaf(v1, c1.y, v0 * c1.x)));
      const float s2 = fmaf(v3, c2.w, fmaf(v2, c2.z, fmaf(v1, c2.y, v0 * c2.x)));
      const float s3 = fmaf(v3, c3.w, fmaf(v2, c3.z, fmaf(v1, c3.y, v0 * c3.x)));
      if (s0 > best) { best = s0; bk = k0; }
      if (s1 > best) { best = s1; bk = k1; }
      if (s2 > best) { best = s2; bk = k2; }
      if (s3 > best) { best = s3; bk = k3; }
      if (kk.x & 0x8000u) break;
      e += 4;
    }
  }
  const int pf = (int)(((float)bk + 0.5f) * inv_S);
  sidx = bk - pf * S;
  prim = L.nm[gp * 24 + pf];
  return true;
}

// Bytes of shared memory a kernel needs for a table of n cells per axis, n_cells stored cells and n_cand candidates.
__host__ __device__ inline size_t lut_smem_bytes(int n, int n_cells, int n_cand) {
  return (size_t)n * n * 4 + (((size_t)n_cells * 2 + 15) & ~(size_t)15) + (((size_t)n_cand * 2 + 15) & ~(size_t)15) + 576;
}
// Copy head h's table into shared memory at `dst` (all threads of the CTA; the caller synchronises) and return the view.
__device__ __forceinline__ LutView lut_to_smem(const unsigned char* __restrict__ lut, int h, unsigned char* dst,
                                               const Mul24& nm) {
  const uint32_t* gh = reinterpret_cast<const uint32_t*>(lut);
  const int n = (int)gh[0], n_cells = (int)gh[1];
  const unsigned char* head = lut + kLutOffHeads + (size_t)h * kLutHeadBytes;
  const uint32_t total = reinterpret_cast<const uint32_t*>(head)[0];
  uint32_t* rows = reinterpret_cast<uint32_t*>(dst);
  uint16_t* cells = reinterpret_cast<uint16_t*>(dst + (size_t)n * n * 4);
  uint16_t* cands = reinterpret_cast<uint16_t*>(dst + (size_t)n * n * 4 + (((size_t)n_cells * 2 + 15) & ~(size_t)15));
  uint8_t* snm = reinterpret_cast<uint8_t*>(cands) + (((size_t)total * 2 + 15) & ~(size_t)15);
  const uint32_t* grows = reinterpret_cast<const uint32_t*>(lut + kLutOffRows);
  for (int i = threadIdx.x; i < n * n; i += blockDim.x) rows[i] = grows[i];
  const uint32_t* gc = reinterpret_cast<const uint32_t*>(head + 16);
  for (int i = threadIdx.x; i < (n_cells + 1) / 2; i += blockDim.x) reinterpret_cast<uint32_t*>(cells)[i] = gc[i];
  const uint32_t* gd = reinterpret_cast<const uint32_t*>(head + 16 + (size_t)kLutCellCap * 2);
  for (uint32_t i = threadIdx.x; i < (total + 1) / 2; i += blockDim.x) reinterpret_cast<uint32_t*>(cands)[i] = gd[i];
  for (int i = threadIdx.x; i < 576; i += blockDim.x) snm[i] = nm.v[i / 24][i % 24];
  LutView L;
  L.rows = rows; L.cells = cells; L.cands = cands; L.nm = snm; L.n = n; L.hn = 0.5f * (float)n;
  return L;
}
// The same table read in place from global memory (small calls).
__device__ __forceinline__ LutView lut_global(const unsigned char* __restrict__ lut, int h, const uint8_t* nm) {
  const uint32_t* gh = reinterpret_cast<const uint32_t*>(lut);
  const unsigned char* head = lut + kLutOffHeads + (size_t)h * kLutHeadBytes;
  LutView L;
  L.rows = reinterpret_cast<const uint32_t*>(lut + kLutOffRows);
  L.cells = reinterpret_cast<const uint16_t*>(head + 16);
  L.cands = reinterpret_cast<const uint16_t*>(head + 16 + (size_t)kLutCellCap * 2);
  L.nm = nm; L.n = (int)gh[0]; L.hn = 0.5f * (float)L.n;
  return L;
}
__device__ __forceinline__ bool lut_head_valid(const unsigned char* __restrict__ lut, int h) {
  return reinterpret_cast<const uint32_t*>(lut + kLutOffHeads + (size_t)h * kLutHeadBytes)[1] == 1u;
}

template <bool LUT>
__global__ void __launch_bounds__(kEncThreads)
encode_main_kernel(EncGeom g, const void* __restrict__ x, const float* __restrict__ qs_all, hqmq_packed dst,
                   int t_start, uint32_t* __restrict__ hist, Maps24 maps, const float* __restrict__ joint_all,
                   const unsigned char* __restrict__ lut, Mul24 nmul) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float4* qs = reinterpret_cast<float4*>(smem_raw);
  uint32_t* rows = reinterpret_cast<uint32_t*>(qs + g.S);            // [warps][tpw][kMaxRowWords]
  uint32_t* shist = rows + kEncWarps * g.tpw * kMaxRowWords;          // [kHistBins]
  float4* sjoint = reinterpret_cast<float4*>(shist + kHistBins);      // LUT: [24 S], then the table of the head

  const int bh = blockIdx.y;
  const int h = bh % g.H, b = bh / g.H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < g.S; i += blockDim.x) qs[i] = reinterpret_cast<const float4*>(qs_all)[(int64_t)h * g.S + i];
  if (hist) for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) shist[i] = 0;
  bool use_lut = false;
  LutView L = {};
  if constexpr (LUT) {
    use_lut = lut_head_valid(lut, h);
    if (use_lut) {
      for (int i = threadIdx.x; i < 24 * g.S; i += blockDim.x) sjoint[i] = reinterpret_cast<const float4*>(joint_all)[(int64_t)h * 24 * g.S + i];
      L = lut_to_smem(lut, h, reinterpret_cast<unsigned char*>(sjoint + 24 * g.S), nmul);
    }
  }
  const float inv_S = 1.0f / (float)g.S;
  __syncthreads();

  const int sub = lane / g.npl, c = lane % g.npl;
  const int rw = dst.row_bytes >> 2;
  const int cb = g.ib + g.rbits;
  uint32_t* myrow = rows + (warp * g.tpw + sub) * kMaxRowWords;
  const int tok_per_iter = kEncWarps * g.tpw;
  const int t_block0 = blockIdx.x * tok_per_iter * kEncIters;

  // the chunk of the next iteration is loaded before the current one is searched
  float vn[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const int t = t_block0 + warp * g.tpw + sub;
    if (t < g.T_new && c < g.n) load_chunk(x, b * g.xs_b + h * g.xs_h + t * g.xs_t + 4 * c, g.x_dtype, vn);
  }
  for (int it = 0; it < kEncIters; ++it) {
    const int t = t_block0 + it * tok_per_iter + warp * g.tpw + sub;
    const bool tok_ok = t < g.T_new;
    const bool active = tok_ok && c < g.n;
    float v[4] = {vn[0], vn[1], vn[2], vn[3]};
    vn[0] = vn[1] = vn[2] = vn[3] = 0.f;
    if (it + 1 < kEncIters) {
      const int t2 = t + tok_per_iter;
      if (t2 < g.T_new && c < g.n) load_chunk(x, b * g.xs_b + h * g.xs_h + t2 * g.xs_t + 4 * c, g.x_dtype, vn);
    }
    const float nrm = chunk_norm(v);
    const float radius = fmaxf(nrm, 1e-8f);
    float rmax = active ? radius : 0.f;
    for (int o = g.npl >> 1; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
    rmax = fmaxf(rmax, 1e-8f);
    const float scale = __fdiv_rn(rmax, (float)g.qmax);
    float rqf = rintf(__fdiv_rn(radius, scale));
    rqf = fminf(fmaxf(rqf, 0.f), (float)g.qmax);

    for (int w = lane; w < g.tpw * kMaxRowWords; w += 32) rows[warp * g.tpw * kMaxRowWords + w] = 0;
    __syncwarp();
    if (active) {
      // the nearest codeword does not depend on the length of the chunk: search with a cheaply
      // normalised copy (keeps the values in range) instead of the reference's exact x / radius
      const float inv_r = __frcp_rn(radius);
      const float u0 = v[0] * inv_r, u1 = v[1] * inv_r, u2 = v[2] * inv_r, u3 = v[3] * inv_r;
      int s, au;
      if (!(LUT && use_lut && search_fold24(sjoint, L, g.S, inv_S, u0, u1, u2, u3, au, s)))
        au = maps.ref_to_native[search_exhaustive(qs, g.S, u0, u1, u2, u3, s)];
      const uint32_t ni = (uint32_t)((((au >> 3) * g.S + s) << 3) | (au & 7));
      const uint32_t f = ni | ((uint32_t)rqf << g.ib);
      const int bit = c * cb, w = bit >> 5, sh = bit & 31;
      atomicOr(&myrow[w], f << sh);
      if (sh + cb > 32) atomicOr(&myrow[w + 1], f >> (32 - sh));
      if (hist) atomicAdd(&shist[__float_as_uint(nrm) >> 21], 1u);
    }
    __syncwarp();
    if (tok_ok) {
      const int64_t row = (int64_t)bh * dst.T_cap + t_start + t;
      uint32_t* out = reinterpret_cast<uint32_t*>(dst.codes + row * dst.row_bytes);
      for (int w = c; w < rw; w += g.npl) out[w] = myrow[w];
      if (c == 0) {
        store_scale(dst, row, rmax);
        if (dst.flags) dst.flags[row] = 0u;
      }
    }
    __syncwarp();
  }
  if (hist) {
    __syncthreads();
    uint32_t* gh = hist + (int64_t)h * 3 * 2 * kHistBins;  // level 0, query 0
    for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) {
      uint32_t cnt = shist[i];
      if (cnt) atomicAdd(&gh[i], cnt);
    }
  }
}

// ---- small calls (decode-time appends) ------------------------------------------------------------------
// One CTA per head does the whole call: norms, per-token scale, nearest codeword (tables read straight from
// global memory: they sit in L2 and a handful of chunks per thread do not pay for staging them), the exact
// median by rank counting in shared memory, flags, packed rows.  It replaces the main pass, the three select
// levels and the flag pass by one launch when a head has at most kSmallMax chunks in the call; the offset
// scan and the side-plane kernel follow as usual.  Same arithmetic as the large-call kernels.
constexpr int kSmallMax = 2048;          // chunks per head and call
constexpr int kSmallThreads = 1024;
constexpr int kSmallTok = 512;           // tokens per head and call (kSmallMax / 4 chunks)

// (the body is shared by the kernel of one tensor and by the kernel that appends K and V of a layer in one launch)
__device__ __forceinline__ void
encode_small_body(const EncGeom& g, const void* __restrict__ x, const float* __restrict__ qs_all, const hqmq_packed& dst,
                  int t_start, const Maps24& maps, const float* __restrict__ joint_all, const unsigned char* __restrict__ lut,
                  const uint8_t* __restrict__ nmul_dev, float C, float* __restrict__ med_out, float quantile) {
  __shared__ uint32_t keys[kSmallMax];                    // norm bits of every chunk of the head
  __shared__ uint32_t tokmax[kSmallTok];                  // bits of the largest radius of a token
  __shared__ uint32_t tokflags[kSmallTok];
  __shared__ uint32_t rows[kSmallTok / 8][kMaxRowWords];   // packed rows, 64 tokens at a time
  const int h = blockIdx.x;
  const int n = g.n, per_b = g.T_new * n;                 // chunks of one batch entry
  const int N = g.B * per_b, n_tok = g.B * g.T_new;
  const int S = g.S;
  const float inv_S = 1.0f / (float)S;
  const bool med = C > 0.f;
  const float qmaxf = (float)g.qmax;
  for (int i = threadIdx.x; i < n_tok; i += blockDim.x) { tokmax[i] = 0u; tokflags[i] = 0u; }
  __syncthreads();

  const bool use_lut = lut && lut_head_valid(lut, h);
  LutView L = {};
  if (use_lut) L = lut_global(lut, h, nmul_dev);
  const float4* joint = reinterpret_cast<const float4*>(joint_all) + (int64_t)h * 24 * S;
  const float4* qs = reinterpret_cast<const float4*>(qs_all) + (int64_t)h * S;

  // ---- phase A: norms, token maxima, nearest codewords ------------------------------------------------------
  float nrm[2], radius[2];
  uint32_t ni[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int i = threadIdx.x + k * kSmallThreads;
    nrm[k] = 0.f; radius[k] = 0.f; ni[k] = 0u;
    if (i < N) {
      const int b = i / per_b, r = i - b * per_b, t = r / n, c = r - t * n;
      float v[4];
      load_chunk(x, b * g.xs_b + h * g.xs_h + t * g.xs_t + 4 * c, g.x_dtype, v);
      nrm[k] = chunk_norm(v);
      radius[k] = fmaxf(nrm[k], 1e-8f);
      keys[i] = __float_as_uint(nrm[k]);
      atomicMax(&tokmax[b * g.T_new + t], __float_as_uint(radius[k]));   // positive floats order like their bits
      const float inv_r = __frcp_rn(radius[k]);
      const float u0 = v[0] * inv_r, u1 = v[1] * inv_r, u2 = v[2] * inv_r, u3 = v[3] * inv_r;
      int sidx, au;
      if (!(use_lut && search_fold24(joint, L, S, inv_S, u0, u1, u2, u3, au, sidx)))
        au = maps.ref_to_native[search_exhaustive(qs, S, u0, u1, u2, u3, sidx)];
      ni[k] = (uint32_t)((((au >> 3) * S + sidx) << 3) | (au & 7));
    }
  }
  __syncthreads();

  // ---- phase B: the two middle order statistics: radix select (4 x 8 bits) of the lower one in shared memory,
  // the upper one is the same value or the next larger key ------------------------------------------------------
  float thr = 0.f;
  if (med) {
    __shared__ uint32_t shist[256];
    __shared__ uint32_t s_state[4];       // prefix, rank, keys <= a, smallest key > a
    const QRank qr = quantile_rank((uint64_t)N, quantile);
    const uint32_t lo = (uint32_t)qr.lo, hi = (uint32_t)qr.hi;
    uint32_t prefix = 0u, rank = lo;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (threadIdx.x < 256) shist[threadIdx.x] = 0u;
      __syncthreads();
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int i = threadIdx.x + k * kSmallThreads;
        if (i < N) {
          const uint32_t key = keys[i];
          if (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&shist[(key >> shift) & 0xffu], 1u);
        }
      }
      __syncthreads();
      if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        uint32_t c8[8], mine = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) { c8[q] = shist[lane * 8 + q]; mine += c8[q]; }
        uint32_t incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += v;
        }
        const uint32_t before = incl - mine;
        if (rank >= before && rank < incl) {      // exactly one lane: the rank is below the number of matching keys
          uint32_t acc = before; int digit = lane * 8 + 7;
          bool found = false;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (!found) {
              if (acc + c8[q] > rank) { digit = lane * 8 + q; found = true; }
              else acc += c8[q];
            }
          }
          s_state[0] = prefix | ((uint32_t)digit << shift);
          s_state[1] = rank - acc;
        }
      }
      __syncthreads();
      prefix = s_state[0]; rank = s_state[1];
    }
    const uint32_t a_bits = prefix;
    if (threadIdx.x == 0) { s_state[2] = 0u; s_state[3] = 0xffffffffu; }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = threadIdx.x + k * kSmallThreads;
      if (i < N) {
        const uint32_t key = keys[i];
        if (key <= a_bits) atomicAdd(&s_state[2], 1u);
        else atomicMin(&s_state[3], key);
      }
    }
    __syncthreads();
    const uint32_t b_bits = s_state[2] > hi ? a_bits : s_state[3];
    const float a = __uint_as_float(a_bits), b2 = __uint_as_float(b_bits);
    const float m = hi == lo ? a : quantile_lerp(a, b2, qr.w);
    thr = __fmul_rn(m, C);
    if (threadIdx.x == 0 && med_out) med_out[h] = m;
  }

  // ---- phase C: radius codes, flags -------------------------------------------------------------------------
  uint32_t field[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int i = threadIdx.x + k * kSmallThreads;
    field[k] = 0u;
    if (i < N) {
      const int b = i / per_b, r = i - b * per_b, t = r / n, c = r - t * n;
      const float rmax = fmaxf(__uint_as_float(tokmax[b * g.T_new + t]), 1e-8f);
      const float scale = __fdiv_rn(rmax, qmaxf);
      float rqf = rintf(__fdiv_rn(radius[k], scale));
      rqf = fminf(fmaxf(rqf, 0.f), qmaxf);
      if (med && nrm[k] > thr) {
        atomicOr(&tokflags[b * g.T_new + t], 1u << c);
        rqf = 0.f;          // a flagged chunk is stored in the side buffer: its radius code in the row is 0
      }
      field[k] = ni[k] | ((uint32_t)rqf << g.ib);
    }
  }
  __syncthreads();

  // ---- phase D: packed rows, 64 tokens at a time; scales and flag words ---------------------------------------
  const int cb = g.ib + g.rbits, rw = dst.row_bytes >> 2;
  for (int tok0 = 0; tok0 < n_tok; tok0 += kSmallTok / 8) {
    for (int w = threadIdx.x; w < (kSmallTok / 8) * kMaxRowWords; w += blockDim.x) (&rows[0][0])[w] = 0u;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = threadIdx.x + k * kSmallThreads;
      if (i < N) {
        const int b = i / per_b, r = i - b * per_b, t = r / n, c = r - t * n;
        const int tok = b * g.T_new + t - tok0;
        if (tok >= 0 && tok < kSmallTok / 8) {
          const int bit = c * cb, w = bit >> 5, sh = bit & 31;
          atomicOr(&rows[tok][w], field[k] << sh);
          if (sh + cb > 32) atomicOr(&rows[tok][w + 1], field[k] >> (32 - sh));
        }
      }
    }
    __syncthreads();
    const int cnt = min(kSmallTok / 8, n_tok - tok0);
    for (int w = threadIdx.x; w < cnt * rw; w += blockDim.x) {
      const int tok = tok0 + w / rw, ww = w - (w / rw) * rw;
      const int b = tok / g.T_new, t = tok - b * g.T_new;
      const int64_t row = ((int64_t)b * g.H + h) * dst.T_cap + t_start + t;
      reinterpret_cast<uint32_t*>(dst.codes + row * dst.row_bytes)[ww] = rows[tok - tok0][ww];
    }
    __syncthreads();
  }
  for (int tok = threadIdx.x; tok < n_tok; tok += blockDim.x) {
    const int b = tok / g.T_new, t = tok - b * g.T_new;
    const int64_t row = ((int64_t)b * g.H + h) * dst.T_cap + t_start + t;
    store_scale(dst, row, fmaxf(__uint_as_float(tokmax[tok]), 1e-8f));
    if (dst.flags) dst.flags[row] = tokflags[tok];
  }
}

// Everything one tensor of a small call needs; two of them make the K + V append of a layer.
struct SmallArgs {
  EncGeom g;
  const void* x;
  const float* qs;
  hqmq_packed dst;
  int t_start;
  const float* joint;
  const unsigned char* lut;
  const uint8_t* nmul;
  float C;
  float* med_out;
  float quantile;
  uint32_t* status;     // first word of the tensor's workspace: cleared here, set by scan_kernel on an overflow
  int blk0, nblk, scan, payload, side;
};
struct SmallPair { SmallArgs t[2]; Maps24 maps; };

__global__ void __launch_bounds__(kSmallThreads) encode_small_kernel(SmallArgs a, Maps24 maps) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *a.status = 0u;
  encode_small_body(a.g, a.x, a.qs, a.dst, a.t_start, maps, a.joint, a.lut, a.nmul, a.C, a.med_out, a.quantile);
}

// ---- main pass for the common geometry ------------------------------------------------------------------
// 32 chunks per token, 16-bit input, look-up-table search, compile-time field layout: one warp per token,
// one lane per chunk, no run-time geometry in the loop.  Results are the ones encode_main_kernel gives.
constexpr int kEnc32Threads = 1024;   // one CTA per SM (the tables fill half of shared memory): 32 warps hide the search latency
constexpr int kEnc32Warps = kEnc32Threads / 32;
// Bracket mode (BR): a two-level select over a sample of the tokens has predicted the threshold statistic to a
// relative 2^-13; the main pass then does everything that needs x in its one read.  Per head, `bp` holds a range
// [R_lo, R_hi] of norm bits around the predicted statistic (+-1 %) and the bounds thr_lo / thr_hi of the threshold
// that follow from it.  A chunk above thr_hi is flagged here (radius code 0, bit in the token's flag word), a chunk
// at or below thr_lo is not, the few in between are listed for the fix-up; the norms inside the range are appended
// to a list (one region per CTA) and the norms below it are counted, from which list_select_kernel takes the exact
// order statistics -- and finds out whether the prediction held: if not, it raises the gate word and the
// multi-pass kernels, which otherwise return at once, redo the call.
struct BracketArgs {
  const uint32_t* bp;       // [H][8]: R_lo, R_hi, thr_lo, thr_hi (float bits), norms below R_lo, ...
  uint32_t* bp_count;       // same array, for the atomics
  uint32_t* band;           // [H][kBandWords]: word 2 counts the undecided chunks
  uint32_t* und;            // [H][kUndCap] undecided chunks
  uint32_t* rcnt;           // [regions] norms appended per region (may exceed rcap: the list then overflowed)
  uint32_t* rlist;          // [regions][rcap]
  uint32_t* histA;          // [H][kHistBins] top digit of (norm bits - R_lo) of the norms inside the range
  int rcap, und_cap;
  const uint32_t* run_if;   // multi-pass (non-bracket) launch: return unless this word is non-zero (nullptr: run)
};
constexpr int kBpWords = 16;

template <int DT, int IB, int RB, bool BR>
__global__ void __launch_bounds__(kEnc32Threads, 1)
encode_main32_kernel(EncGeom g, const uint16_t* __restrict__ x, const float* __restrict__ qs_all, hqmq_packed dst,
                     int t_start, uint32_t* __restrict__ hist, Maps24 maps, const float* __restrict__ joint_all,
                     const unsigned char* __restrict__ lut, Mul24 nmul, int iters,
                     const uint32_t* __restrict__ sel_s, BracketArgs br) {
  if (!BR && br.run_if && *br.run_if == 0u) return;
  __shared__ uint32_t s_below, s_rcount;
  constexpr int CB = IB + RB;
  constexpr int RW = 32 * CB / 32;                       // words per row
  constexpr float qmaxf = (float)((1 << RB) - 1);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float4* qs = reinterpret_cast<float4*>(smem_raw);
  uint32_t* rows = reinterpret_cast<uint32_t*>(qs + g.S);            // [warps][kMaxRowWords]
  uint32_t* shist = rows + kEnc32Warps * kMaxRowWords;                  // [kHistBins]
  uint32_t* sh1 = shist + kHistBins;                                  // [2][kHistBins]: next digit inside the predicted bins
  float4* sjoint = reinterpret_cast<float4*>(sh1 + 2 * kHistBins);    // [24 S], then the look-up table of the head

  const int bh = blockIdx.y;
  const int h = bh % g.H, b = bh / g.H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = g.S;
  for (int i = threadIdx.x; i < S; i += blockDim.x) qs[i] = reinterpret_cast<const float4*>(qs_all)[(int64_t)h * S + i];
  if (hist || BR) for (int i = threadIdx.x; i < 3 * kHistBins; i += blockDim.x) shist[i] = 0;   // shist and sh1
  for (int i = threadIdx.x; i < 24 * S; i += blockDim.x) sjoint[i] = reinterpret_cast<const float4*>(joint_all)[(int64_t)h * 24 * S + i];
  const LutView L = lut_to_smem(lut, h, reinterpret_cast<unsigned char*>(sjoint + 24 * S), nmul);
  const float inv_S = 1.0f / (float)S;
  // Bins (norm bits 31:21) that a sample of the call says hold the two middle order statistics: their next
  // 11-bit digit is histogrammed here too, which spares a pass over x when the sample was right.
  const uint32_t pb0 = sel_s ? sel_s[h * 8 + 0] >> 21 : 0xffffffffu, pb1 = sel_s ? sel_s[h * 8 + 2] >> 21 : 0xffffffffu;
  uint32_t r_lo = 0u, r_hi = 0u, n_below = 0u, s1 = 0u;
  float thr_lo = 0.f, thr_hi = 0.f;
  const int region = blockIdx.y * gridDim.x + blockIdx.x;
  if constexpr (BR) {
    r_lo = br.bp[h * kBpWords + 0]; r_hi = br.bp[h * kBpWords + 1];
    thr_lo = __uint_as_float(br.bp[h * kBpWords + 2]); thr_hi = __uint_as_float(br.bp[h * kBpWords + 3]);
    s1 = br.bp[h * kBpWords + 5];
    if (threadIdx.x == 0) { s_below = 0u; s_rcount = 0u; }
  }
  __syncthreads();

  uint32_t* myrow = rows + warp * kMaxRowWords;
  const int t_block0 = blockIdx.x * kEnc32Warps * iters;
  const uint16_t* xp = x + b * g.xs_b + h * g.xs_h + 4 * lane;
  int t = t_block0 + warp;
  uint2 raw_n = make_uint2(0u, 0u);
  if (t < g.T_new) raw_n = *reinterpret_cast<const uint2*>(xp + (int64_t)t * g.xs_t);
  for (int it = 0; it < iters && t < g.T_new; ++it, t += kEnc32Warps) {
    const uint2 raw = raw_n;
    if (it + 1 < iters && t + kEnc32Warps < g.T_new)
      raw_n = *reinterpret_cast<const uint2*>(xp + (int64_t)(t + kEnc32Warps) * g.xs_t);
    float v[4];
    v[0] = bits16_to_float(raw.x & 0xffff, DT); v[1] = bits16_to_float(raw.x >> 16, DT);
    v[2] = bits16_to_float(raw.y & 0xffff, DT); v[3] = bits16_to_float(raw.y >> 16, DT);
    const float nrm = chunk_norm(v);
    const float radius = fmaxf(nrm, 1e-8f);
    float rmax = radius;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
    {
      const float other = __shfl_xor_sync(0xffffffffu, rmax, 16);
      if (!g.pair16) rmax = fmaxf(rmax, other);       // (pairs: each half-warp is a token of its own)
    }
    const float scale = __fdiv_rn(rmax, qmaxf);
    // radius code: the quotient is first taken with an approximate reciprocal; only a lane whose quotient
    // lies close to a rounding boundary repeats it with the IEEE division the contract names
    float quo = radius * rcp_approx(scale);
    float rqf = rintf(quo);
    if (fabsf(quo - rqf) > 0.499f) rqf = rintf(__fdiv_rn(radius, scale));
    rqf = fminf(fmaxf(rqf, 0.f), qmaxf);
    uint32_t flag_word = 0u;
    if constexpr (BR) {
      const uint32_t key = __float_as_uint(nrm);
      const bool certain = nrm > thr_hi;
      if (certain) rqf = 0.f;                       // a flagged chunk's values live in the side buffer
      flag_word = __ballot_sync(0xffffffffu, certain);
      if (!certain && nrm > thr_lo) {               // rare: settled against the exact threshold afterwards
        const uint32_t pos = atomicAdd(&br.band[h * kBandWords + 2], 1u);
        if (pos < (uint32_t)br.und_cap)
          br.und[(int64_t)h * br.und_cap + pos] =
              g.pair16 ? (uint32_t)(((int64_t)b * (2 * g.T_new) + 2 * t + (lane >> 4)) * 32 + (lane & 15))
                       : (uint32_t)(((int64_t)b * g.T_new + t) * 32 + lane);
      }
      n_below += __popc(__ballot_sync(0xffffffffu, key < r_lo));       // (every lane keeps the warp's count)
      const bool in_range = key >= r_lo && key <= r_hi;
      const uint32_t m = __ballot_sync(0xffffffffu, in_range);
      if (m) {
        uint32_t base = 0u;
        if (lane == 0) base = atomicAdd(&s_rcount, (uint32_t)__popc(m));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (in_range) {
          const uint32_t pos = base + __popc(m & ((1u << lane) - 1u));
          if (pos < (uint32_t)br.rcap) br.rlist[(int64_t)region * br.rcap + pos] = key;
          atomicAdd(&shist[((key - r_lo) >> s1) & (kHistBins - 1)], 1u);
        }
      }
    }

    // ---- nearest codeword ---------------------------------------------------------------------------
    // (the nearest codeword does not depend on the chunk's length: a cheaply normalised copy keeps the
    // values in range)
    const float inv_r = rcp_approx(radius);
    const float u0 = v[0] * inv_r, u1 = v[1] * inv_r, u2 = v[2] * inv_r, u3 = v[3] * inv_r;
    int au, sidx;
    if (!search_fold24(sjoint, L, S, inv_S, u0, u1, u2, u3, au, sidx)) {
      // zero direction (every similarity is 0, the first index wins) or a cell without a list
      int p = 0; sidx = 0;
      if (fmaxf(fmaxf(fabsf(u0), fabsf(u1)), fmaxf(fabsf(u2), fabsf(u3))) > 0.f) p = search_exhaustive(qs, S, u0, u1, u2, u3, sidx);
      au = maps.ref_to_native[p];
    }
    const uint32_t ni = (uint32_t)((((au >> 3) * S + sidx) << 3) | (au & 7));
    const uint32_t f = ni | ((uint32_t)rqf << IB);

    // ---- packed row, scale, flag word ---------------------------------------------------------------------
    const int64_t row = (int64_t)bh * dst.T_cap + t_start + (g.pair16 ? 2 * t : t);   // (pairs: two rows, contiguous)
    uint32_t* out = reinterpret_cast<uint32_t*>(dst.codes + row * dst.row_bytes);
    if constexpr (CB == 16) {
      const uint32_t other = __shfl_xor_sync(0xffffffffu, f, 1);
      if (!(lane & 1)) out[lane >> 1] = f | (other << 16);
    } else {
      if (lane < RW) myrow[lane] = 0;
      __syncwarp();
      const int bit = lane * CB, w = bit >> 5, sh = bit & 31;
      atomicOr(&myrow[w], f << sh);
      if (sh + CB > 32) atomicOr(&myrow[w + 1], f >> (32 - sh));
      __syncwarp();
      if (lane < RW) out[lane] = myrow[lane];
      __syncwarp();
    }
    if (lane == 0 || (g.pair16 && lane == 16)) {
      const int half = lane >> 4;
      store_scale(dst, row + half, rmax);
      if (dst.flags) dst.flags[row + half] = g.pair16 ? (half ? flag_word >> 16 : flag_word & 0xffffu) : flag_word;
    }
    if (!BR && hist) {
      const uint32_t key = __float_as_uint(nrm), top = key >> 21;
      atomicAdd(&shist[top], 1u);
      if (top == pb0) atomicAdd(&sh1[(key >> 10) & 0x7ffu], 1u);
      else if (top == pb1) atomicAdd(&sh1[kHistBins + ((key >> 10) & 0x7ffu)], 1u);
    }
  }
  if constexpr (BR) {
    if (lane == 0 && n_below) atomicAdd(&s_below, n_below);
    __syncthreads();
    if (threadIdx.x == 0) {
      if (s_below) atomicAdd(&br.bp_count[h * kBpWords + 4], s_below);
      br.rcnt[region] = s_rcount;
      if (s_rcount > (uint32_t)br.rcap) atomicOr(&br.bp_count[h * kBpWords + 10], 1u);
    }
    uint32_t* gA = br.histA + (int64_t)h * kHistBins;
    for (int i = threadIdx.x; i < kHistBins; i += blockDim.x)
      if (shist[i]) atomicAdd(&gA[i], shist[i]);
  }
  if (!BR && hist) {
    __syncthreads();
    uint32_t* gh = hist + (int64_t)h * 3 * 2 * kHistBins;  // level 0, query 0
    for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) {
      uint32_t cnt = shist[i];
      if (cnt) atomicAdd(&gh[i], cnt);
    }
    if (sel_s) {
      uint32_t* g1 = gh + 2 * kHistBins;                   // level 1, both queries
      const bool same = pb0 == pb1;
      for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) {
        const uint32_t c0 = sh1[i], c1 = same ? c0 : sh1[kHistBins + i];
        if (c0) atomicAdd(&g1[i], c0);
        if (c1) atomicAdd(&g1[kHistBins + i], c1);
      }
    }
  }
}

// ---- Med3x: radix select of the two middle order statistics ------------------------------
// Level 0 histogram (bits 31:21) is accumulated by encode_main_kernel into query slot 0.
__global__ void __launch_bounds__(256)
select_kernel(uint32_t* __restrict__ hist, uint32_t* __restrict__ sel, int level, uint64_t N, float C,
              float* __restrict__ med_out, uint32_t* __restrict__ band, const uint32_t* __restrict__ sel_s,
              const uint32_t* __restrict__ hist_fb, float quantile, const uint32_t* __restrict__ gate, int gate_want) {
  __shared__ uint64_t wtot[8];
  if (gate && (*gate != 0u) != (gate_want != 0)) return;   // (this launch belongs to the other of the two paths)

  const int h = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;   // launched with 256 threads
  uint32_t* st = sel + h * 8;
  // level 1 with a sampled prediction: the main pass filled the level-1 histograms if the sample named the
  // right bins, else hist32_kernel filled the fallback ones
  const bool use_fb = level == 1 && sel_s && !(sel_s[h * 8 + 0] == st[0] && sel_s[h * 8 + 2] == st[2]);
  const QRank qr = quantile_rank(N, quantile);
  const uint64_t lo = qr.lo, hi = qr.hi;
  uint32_t* hl = hist + ((int64_t)h * 3 + level) * 2 * kHistBins;
  const int shift = level == 0 ? 21 : level == 1 ? 10 : 0;
  const int bins = level == 2 ? 1024 : kHistBins;
  const int per = bins / 256;         // bins per thread: 8 or 4
  for (int q = 0; q < 2; ++q) {
    const uint64_t rank = level == 0 ? (q == 0 ? lo : hi) : st[2 * q + 1];
    const uint32_t prefix = level == 0 ? 0u : st[2 * q];
    // level 0 has one histogram (slot 0); deeper levels have one per query
    const uint32_t* hq = use_fb ? hist_fb + ((int64_t)h * 2 + q) * kHistBins : hl + (level == 0 ? 0 : q * kHistBins);
    uint32_t cnt[8];
#pragma unroll
    for (int i = 0; i < 8; i += 4) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (i < per) v = *reinterpret_cast<const uint4*>(hq + tid * per + i);
      cnt[i] = v.x; cnt[i + 1] = v.y; cnt[i + 2] = v.z; cnt[i + 3] = v.w;
    }
    uint64_t mine = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) mine += cnt[i];
    uint64_t incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
      const uint64_t y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    __syncthreads();                  // the previous query's readers of wtot are done
    if (lane == 31) wtot[warp] = incl;
    __syncthreads();
    uint64_t base = 0;
    for (int w = 0; w < warp; ++w) base += wtot[w];
    incl += base;
    const uint64_t before = incl - mine;
    // the thread whose bins hold the rank (the last thread takes an out-of-range rank)
    const bool owner = (rank >= before && rank < incl) || (tid == 255 && rank >= incl);
    if (owner) {
      uint64_t acc = before; int bin = bins - 1;
      bool found = false;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i < per && !found) {
          if (acc + cnt[i] > rank) { bin = tid * per + i; found = true; }
          else acc += cnt[i];
        }
      }
      st[2 * q] = prefix | ((uint32_t)bin << shift);
      st[2 * q + 1] = (uint32_t)(rank - acc);
    }
  }
  __syncthreads();
  if (tid != 0) return;
  if (level == 1 && band) {
    // 22 bits of both order statistics are known: a >= prefix_a, b <= prefix_b | 0x3ff, a <= med <= b, and
    // thr = fl(med * C) is monotone in med, so it lies in [fl(a_lo * C), fl(b_hi * C)]
    band[h * kBandWords + 0] = __float_as_uint(__fmul_rn(__uint_as_float(st[0]), C));
    band[h * kBandWords + 1] = __float_as_uint(__fmul_rn(__uint_as_float(st[2] | 0x3ffu), C));
  }
  if (level == 2) {
    const float a = __uint_as_float(st[0]), b = __uint_as_float(st[2]);
    float med = hi == lo ? a : quantile_lerp(a, b, qr.w);
    const float thr = __fmul_rn(med, C);
    st[4] = st[0]; st[5] = st[2];
    st[6] = __float_as_uint(thr);
    st[7] = __float_as_uint(med);
    if (med_out) med_out[h] = med;
  }
}

// Levels 1 and 2: re-read x, recompute the norms, histogram the next digit of the keys that
// match each query's prefix.
__global__ void __launch_bounds__(256)
hist_kernel(EncGeom g, const void* __restrict__ x, uint32_t* __restrict__ hist, const uint32_t* __restrict__ sel,
            int level) {
  __shared__ uint32_t sh[2][kHistBins];
  const int bh = blockIdx.y;
  const int h = bh % g.H, b = bh / g.H;
  for (int i = threadIdx.x; i < 2 * kHistBins; i += blockDim.x) (&sh[0][0])[i] = 0;
  __syncthreads();
  const uint32_t p0 = sel[h * 8 + 0], p1 = sel[h * 8 + 2];
  // level 0 (used when the histograms of several GPUs are summed between the levels): nothing is fixed yet; a
  // norm has sign bit 0 and `sel` starts zeroed, so comparing bit 31 alone lets every key through
  const int hs = level == 0 ? 31 : level == 1 ? 21 : 10;   // bits already fixed are above hs
  const int ds = level == 0 ? 21 : level == 1 ? 10 : 0;
  const uint32_t dm = level == 2 ? 0x3ffu : 0x7ffu;
  const int64_t total = (int64_t)g.T_new * g.n;
  const int64_t per_block = (total + gridDim.x - 1) / gridDim.x;
  const int64_t i0 = blockIdx.x * per_block, i1 = min(total, i0 + per_block);
  // four independent loads in flight per thread
  for (int64_t i = i0 + threadIdx.x; i < i1; i += 4 * blockDim.x) {
    float v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t iu = i + (int64_t)u * blockDim.x;
      if (iu < i1) {
        int64_t off = b * g.xs_b + h * g.xs_h;
        if (g.xs_t == 4 * g.n) off += iu * 4;     // tokens are contiguous: the (t, chunk) grid is flat
        else { const uint32_t t = (uint32_t)iu / (uint32_t)g.n, c = (uint32_t)iu - t * (uint32_t)g.n; off += (int64_t)t * g.xs_t + 4 * c; }
        load_chunk(x, off, g.x_dtype, v[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (i + (int64_t)u * blockDim.x < i1) {
        const uint32_t key = __float_as_uint(chunk_norm(v[u]));
        const uint32_t dig = (key >> ds) & dm;
        if ((key >> hs) == (p0 >> hs)) atomicAdd(&sh[0][dig], 1u);
        if ((key >> hs) == (p1 >> hs)) atomicAdd(&sh[1][dig], 1u);
      }
    }
  }
  __syncthreads();
  uint32_t* gh = hist + ((int64_t)h * 3 + level) * 2 * kHistBins;
  for (int i = threadIdx.x; i < 2 * kHistBins; i += blockDim.x) {
    uint32_t cnt = (&sh[0][0])[i];
    if (cnt) atomicAdd(&gh[i], cnt);
  }
}

// ---- Med3x passes for the common geometry -----------------------------------------------------------------
// 32 chunks per token (d_head 128), 16-bit inputs, token rows 16-byte aligned: one lane reads two chunks
// (16 bytes), half a warp reads a token, and every thread keeps four such loads in flight.
struct Fast32 {
  const uint16_t* x;
  int64_t xs_b, xs_h, xs_t;
  int H, T_new;
  int pair;      // 1: every "token" here is two consecutive tokens of 16 chunks (d_head 64), see EncGeom::pair16
};
constexpr int kF32Tok = 64;   // tokens per CTA iteration: 8 warps x 2 tokens x 4 loads

template <int DT>
__device__ __forceinline__ void norms_of_two(const uint4& r, float& n0, float& n1) {
  float a[4], b[4];
  a[0] = bits16_to_float(r.x & 0xffff, DT); a[1] = bits16_to_float(r.x >> 16, DT);
  a[2] = bits16_to_float(r.y & 0xffff, DT); a[3] = bits16_to_float(r.y >> 16, DT);
  b[0] = bits16_to_float(r.z & 0xffff, DT); b[1] = bits16_to_float(r.z >> 16, DT);
  b[2] = bits16_to_float(r.w & 0xffff, DT); b[3] = bits16_to_float(r.w >> 16, DT);
  n0 = chunk_norm(a); n1 = chunk_norm(b);
}

template <int DT>
__global__ void __launch_bounds__(256)
hist32_kernel(Fast32 f, uint32_t* __restrict__ hist, const uint32_t* __restrict__ sel, int level,
              const uint32_t* __restrict__ sel_s, uint32_t* __restrict__ hist_fb, const uint32_t* __restrict__ gate, int gate_want) {
  __shared__ uint32_t sh[2][kHistBins];
  if (gate && (*gate != 0u) != (gate_want != 0)) return;   // (this launch belongs to the other of the two paths)

  const int bh = blockIdx.y;
  const int h = bh % f.H, b = bh / f.H;
  // with a sampled prediction this pass is only the fallback: nothing to do when the sample named the right bins
  if (sel_s && sel_s[h * 8 + 0] == sel[h * 8 + 0] && sel_s[h * 8 + 2] == sel[h * 8 + 2]) return;
  for (int i = threadIdx.x; i < 2 * kHistBins; i += blockDim.x) (&sh[0][0])[i] = 0;
  __syncthreads();
  const uint32_t p0 = sel[h * 8 + 0], p1 = sel[h * 8 + 2];
  // level 0 (used when the histograms of several GPUs are summed between the levels): nothing is fixed yet; a
  // norm has sign bit 0 and `sel` starts zeroed, so comparing bit 31 alone lets every key through
  const int hs = level == 0 ? 31 : level == 1 ? 21 : 10;   // bits already fixed are above hs
  const int ds = level == 0 ? 21 : level == 1 ? 10 : 0;
  const uint32_t dm = level == 2 ? 0x3ffu : 0x7ffu;
  const uint32_t q0 = p0 >> hs, q1 = p1 >> hs;
  const bool same = q0 == q1;                            // both order statistics share the prefix: one histogram
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, l16 = lane & 15;
  int per = (f.T_new + gridDim.x - 1) / gridDim.x;
  per = (per + kF32Tok - 1) / kF32Tok * kF32Tok;
  const int t0 = blockIdx.x * per, t1 = min(f.T_new, t0 + per);
  const uint16_t* base = f.x + b * f.xs_b + h * f.xs_h + 8 * l16;
  for (int t = t0 + warp * 2 + (lane >> 4); t < t1; t += kF32Tok) {
    uint4 r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (t + 16 * u < t1) r[u] = *reinterpret_cast<const uint4*>(base + (int64_t)(t + 16 * u) * f.xs_t);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (t + 16 * u < t1) {
        float n[2];
        norms_of_two<DT>(r[u], n[0], n[1]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t key = __float_as_uint(n[e]);
          const uint32_t dig = (key >> ds) & dm, top = key >> hs;
          if (top == q0) atomicAdd(&sh[0][dig], 1u);
          else if (top == q1) atomicAdd(&sh[1][dig], 1u);
        }
      }
    }
  }
  __syncthreads();
  uint32_t* gh = sel_s ? hist_fb + (int64_t)h * 2 * kHistBins : hist + ((int64_t)h * 3 + level) * 2 * kHistBins;
  for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) {
    const uint32_t c0 = sh[0][i], c1 = same ? c0 : sh[1][i];
    if (c0) atomicAdd(&gh[i], c0);
    if (c1) atomicAdd(&gh[kHistBins + i], c1);
  }
}

// Histogram of every kSampleStride-th token: level 0 (norm bits 31:21) predicts the bins of the two order
// statistics before the main pass runs; level 1 (bits 20:10 of the sampled norms inside those bins, `sel_s` holding
// the level-0 result) refines the prediction to 22 bits for the bracket mode of the main pass.
constexpr int kSampleStride = 32;
template <int DT>
__global__ void __launch_bounds__(256)
sample32_kernel(Fast32 f, uint32_t* __restrict__ hist_s, int level, const uint32_t* __restrict__ sel_s) {
  __shared__ uint32_t sh[2][kHistBins];
  const int bh = blockIdx.y;
  const int h = bh % f.H, b = bh / f.H;
  for (int i = threadIdx.x; i < 2 * kHistBins; i += blockDim.x) (&sh[0][0])[i] = 0;
  __syncthreads();
  const uint32_t q0 = level ? sel_s[h * 8 + 0] >> 21 : 0u, q1 = level ? sel_s[h * 8 + 2] >> 21 : 0u;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, l16 = lane & 15;
  const int n_s = (f.T_new + kSampleStride - 1) / kSampleStride;       // sampled tokens of this (b, h)
  const uint16_t* base = f.x + b * f.xs_b + h * f.xs_h + 8 * l16;
  for (int k = blockIdx.x * 16 + warp * 2 + (lane >> 4); k < n_s; k += gridDim.x * 16) {
    const uint4 r = *reinterpret_cast<const uint4*>(base + (int64_t)k * kSampleStride * f.xs_t);
    float n[2];
    norms_of_two<DT>(r, n[0], n[1]);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const uint32_t key = __float_as_uint(n[e]);
      if (level == 0) atomicAdd(&sh[0][key >> 21], 1u);
      else if ((key >> 21) == q0) atomicAdd(&sh[0][(key >> 10) & 0x7ffu], 1u);
      else if ((key >> 21) == q1) atomicAdd(&sh[1][(key >> 10) & 0x7ffu], 1u);
    }
  }
  __syncthreads();
  // laid out like the full histograms: level 0 has one slot, level 1 one per order statistic
  uint32_t* gh = hist_s + ((int64_t)h * 3 + level) * 2 * kHistBins;
  const bool same = q0 == q1;
  for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) {
    const uint32_t c0 = sh[0][i];
    if (c0) atomicAdd(&gh[i], c0);
    if (level) {
      const uint32_t c1 = same ? c0 : sh[1][i];
      if (c1) atomicAdd(&gh[kHistBins + i], c1);
    }
  }
}

// Bracket of the main pass from the sample's two-level select: the order statistics a <= b of the whole call are
// expected inside [R_lo, R_hi] = [a_s (1 - delta), b_s (1 + delta)], where a_s / b_s are the sample's statistics known to
// 22 bits (low bits 0 / all ones).  The threshold is fl(lerp(a, b, w) * C) with lerp(a, b, w) in [a, b] and fl
// monotone, so it then lies in [fl(R_lo * C), fl(R_hi * C)].  Whether the expectation held is checked exactly by
// list_select_kernel.
__global__ void bracket_kernel(const uint32_t* __restrict__ sel_s, float C, float delta, int H, uint32_t* __restrict__ bp,
                               uint32_t* __restrict__ band) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  const float a_s = __uint_as_float(sel_s[h * 8 + 0]), b_s = __uint_as_float(sel_s[h * 8 + 2] | 0x3ffu);
  const float r_lo = __fmul_rn(a_s, 1.f - delta), r_hi = __fmul_rn(b_s, 1.f + delta);
  bp[h * kBpWords + 0] = __float_as_uint(r_lo);
  bp[h * kBpWords + 1] = __float_as_uint(r_hi);
  bp[h * kBpWords + 2] = __float_as_uint(__fmul_rn(r_lo, C));
  bp[h * kBpWords + 3] = __float_as_uint(__fmul_rn(r_hi, C));
  // top digit of (norm bits - R_lo): 2048 bins of 2^s1 keys cover the range (a range wider than 2^22 keys -- a
  // statistic next to zero -- is left to the multi-pass path)
  const uint32_t width = __float_as_uint(r_hi) - __float_as_uint(r_lo);
  const int bits = 32 - __clz(width | 1u);
  bp[h * kBpWords + 5] = (uint32_t)(bits > 11 ? bits - 11 : 0);
  band[h * kBandWords + 0] = bp[h * kBpWords + 2];
  band[h * kBandWords + 1] = bp[h * kBpWords + 3];
}

// ---- exact order statistics of a head from what the bracket pass left ------------------------------------------
// The pass counted the norms below the range, histogrammed the top digit of (norm bits - R_lo) for the norms inside
// it (`histA`, 2048 bins of 2^s1 keys each) and listed those norms per CTA region.  list_pickA_kernel checks that both
// order statistics fall inside the range (else the prediction failed and the gate word is raised) and names the bin
// of the lower one and the next non-empty bin; list_histB_kernel histograms the low s1 bits of the listed norms
// of those two bins; list_pickB_kernel then has both statistics exactly and writes the select words of the head
// (a, b, threshold, statistic) like the last level of select_kernel.
// bp words: 0 R_lo, 1 R_hi, 2 thr_lo, 3 thr_hi, 4 norms below R_lo, 5 s1, 6 bin of a, 7 next non-empty bin (or ~0),
// 8 rank of a inside its bin, 9 listed norms before the bin of a, 10 a region overflowed
template <int NT>
__device__ __forceinline__ void block_find_rank(const uint32_t* __restrict__ hist, int nbins, uint32_t rank, uint32_t* s_part,
                                                int& bin, uint32_t& before, int& next_bin) {
  // hist in shared or global memory; every thread sums its stretch, thread 0 walks the stretch sums
  const int tid = threadIdx.x, per = (nbins + NT - 1) / NT;
  uint32_t mine = 0;
  for (int i = tid * per; i < min(nbins, (tid + 1) * per); ++i) mine += hist[i];
  s_part[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    uint32_t acc = 0; int t = 0;
    while (t < NT - 1 && acc + s_part[t] <= rank) acc += s_part[t++];
    int i = t * per;
    const int end = min(nbins, (t + 1) * per);
    while (i < end - 1 && acc + hist[i] <= rank) acc += hist[i++];
    int nx = i + 1;
    while (nx < nbins && hist[nx] == 0u) ++nx;
    s_part[NT] = (uint32_t)i; s_part[NT + 1] = acc; s_part[NT + 2] = nx < nbins ? (uint32_t)nx : 0xffffffffu;
  }
  __syncthreads();
  bin = (int)s_part[NT]; before = s_part[NT + 1]; next_bin = (int)s_part[NT + 2];
  __syncthreads();
}

__global__ void __launch_bounds__(256)
list_pickA_kernel(uint32_t* __restrict__ bp, const uint32_t* __restrict__ histA, uint64_t N, float quantile,
                  uint32_t* __restrict__ gate) {
  __shared__ uint32_t s_part[256 + 4];
  __shared__ uint32_t s_tot;
  const int h = blockIdx.x, tid = threadIdx.x;
  const uint32_t* hA = histA + (int64_t)h * kHistBins;
  if (tid == 0) s_tot = 0u;
  __syncthreads();
  uint32_t mine = 0;
  for (int i = tid; i < kHistBins; i += 256) mine += hA[i];
  if (mine) atomicAdd(&s_tot, mine);
  __syncthreads();
  const QRank qr = quantile_rank(N, quantile);
  const uint64_t below = bp[h * kBpWords + 4];
  const bool ok = !bp[h * kBpWords + 10] && bp[h * kBpWords + 5] <= 11u && qr.lo >= below && qr.hi < below + s_tot;
  if (!ok) {
    if (tid == 0) atomicExch(gate, 1u);
    return;
  }
  int bin, next_bin; uint32_t before;
  block_find_rank<256>(hA, kHistBins, (uint32_t)(qr.lo - below), s_part, bin, before, next_bin);
  if (tid == 0) {
    bp[h * kBpWords + 6] = (uint32_t)bin;
    bp[h * kBpWords + 7] = (uint32_t)next_bin;
    bp[h * kBpWords + 8] = (uint32_t)(qr.lo - below) - before;
    bp[h * kBpWords + 9] = before;
  }
}

// grid = the main pass's grid (one CTA per list region)
__global__ void __launch_bounds__(256)
list_histB_kernel(const uint32_t* __restrict__ bp, const uint32_t* __restrict__ rcnt, const uint32_t* __restrict__ rlist, int rcap,
                  int H, uint32_t* __restrict__ histB, const uint32_t* __restrict__ gate) {
  if (*gate) return;
  const int bh = blockIdx.y, h = bh % H;
  const int region = blockIdx.y * gridDim.x + blockIdx.x;
  const uint32_t r_lo = bp[h * kBpWords + 0], s1 = bp[h * kBpWords + 5];
  const uint32_t bin0 = bp[h * kBpWords + 6], bin1 = bp[h * kBpWords + 7];
  const uint32_t lowmask = (1u << s1) - 1u;
  uint32_t c = rcnt[region];
  if (c > (uint32_t)rcap) c = rcap;
  const uint32_t* keys = rlist + (int64_t)region * rcap;
  uint32_t* hB = histB + (int64_t)h * 2 * kHistBins;
  // (the bins hold few keys: straight to the global histograms)
  for (uint32_t i0 = threadIdx.x; i0 < c; i0 += 4 * 256) {
    uint32_t k[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) k[u] = i0 + u * 256 < c ? keys[i0 + u * 256] : 0xffffffffu;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (i0 + u * 256 < c) {
        const uint32_t off = k[u] - r_lo, top = off >> s1;
        if (top == bin0) atomicAdd(&hB[off & lowmask], 1u);
        else if (top == bin1) atomicAdd(&hB[kHistBins + (off & lowmask)], 1u);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
list_pickB_kernel(const uint32_t* __restrict__ bp, const uint32_t* __restrict__ histB, uint64_t N, float C, float quantile,
                  uint32_t* __restrict__ sel, float* __restrict__ med_out, const uint32_t* __restrict__ gate) {
  __shared__ uint32_t s_part[256 + 4];
  if (*gate) return;
  const int h = blockIdx.x, tid = threadIdx.x;
  const uint32_t r_lo = bp[h * kBpWords + 0], s1 = bp[h * kBpWords + 5];
  const uint32_t bin0 = bp[h * kBpWords + 6], bin1 = bp[h * kBpWords + 7], rank = bp[h * kBpWords + 8];
  const uint32_t* hB = histB + (int64_t)h * 2 * kHistBins;
  const int nb = 1 << s1;
  int bin, next_bin; uint32_t before;
  block_find_rank<256>(hB, nb, rank, s_part, bin, before, next_bin);
  // smallest key of the next non-empty top bin (the upper statistic when a is the last key of its bin)
  int first1 = 0, dummy_n; uint32_t dummy_b;
  if (bin1 != 0xffffffffu) block_find_rank<256>(hB + kHistBins, nb, 0u, s_part, first1, dummy_b, dummy_n);
  if (tid == 0) {
    const QRank qr = quantile_rank(N, quantile);
    const uint32_t a_bits = r_lo + (bin0 << s1) + (uint32_t)bin;
    uint32_t b_bits = a_bits;
    if (qr.hi != qr.lo && before + hB[bin] <= rank + 1u) {      // the key after a's run of equal keys
      if (next_bin != -1) b_bits = r_lo + (bin0 << s1) + (uint32_t)next_bin;
      else b_bits = r_lo + (bin1 << s1) + (uint32_t)first1;      // (pickA made sure the statistic exists in the list)
    }
    const float a = __uint_as_float(a_bits), b = __uint_as_float(b_bits);
    const float med = qr.hi == qr.lo ? a : quantile_lerp(a, b, qr.w);
    uint32_t* st = sel + h * 8;
    st[4] = a_bits; st[5] = b_bits;
    st[6] = __float_as_uint(__fmul_rn(med, C));
    st[7] = __float_as_uint(med);
    if (med_out) med_out[h] = med;
  }
}

// Clear the radius code of chunk c in a packed row (atomics: other threads may own neighbouring chunks).
__device__ __forceinline__ void clear_radius(uint32_t* rowp, int c, int ib, int rbits) {
  const int cb = ib + rbits;
  const int lo = c * cb + ib, hi = (c + 1) * cb;   // bit range of the radius code
  const int w0 = lo >> 5, w1 = (hi - 1) >> 5;
  const uint32_t m0 = ~0u << (lo & 31);
  const uint32_t m1 = (hi & 31) ? ~(~0u << (hi & 31)) : ~0u;
  if (w0 == w1) atomicAnd(&rowp[w0], ~(m0 & m1));
  else { atomicAnd(&rowp[w0], ~m0); atomicAnd(&rowp[w1], ~m1); }
}

// Flag a chunk found to be an outlier after the provisional pass.
__device__ __forceinline__ void flag_late(const hqmq_packed& dst, int64_t row, int c, int ib, int rbits) {
  atomicOr(&dst.flags[row], 1u << c);
  clear_radius(reinterpret_cast<uint32_t*>(dst.codes + row * dst.row_bytes), c, ib, rbits);
}

// Last histogram level and the flags in ONE pass over x.  After level 1 the threshold is known to lie in
// [thr_lo, thr_hi] (a relative width of 2^-13): a chunk above thr_hi is an outlier whatever the last ten
// bits of the median turn out to be, a chunk at or below thr_lo is not, and the (normally empty) set in
// between is listed for fixup_list_kernel; if the list overflows, fixup_scan_kernel re-reads x for that head.
// A flagged chunk is stored in the side buffer: its radius code in the packed row becomes 0 so that decoding
// the row contributes nothing for it.
template <int DT>
__global__ void __launch_bounds__(256)
histflags32_kernel(Fast32 f, hqmq_packed dst, int t_start, int ib, int rbits, uint32_t* __restrict__ hist,
                   const uint32_t* __restrict__ sel, uint32_t* __restrict__ band, uint32_t* __restrict__ und,
                   const uint32_t* __restrict__ gate, int gate_want) {
  __shared__ uint32_t sh[2][1024];
  if (gate && (*gate != 0u) != (gate_want != 0)) return;   // (this launch belongs to the other of the two paths)

  const int bh = blockIdx.y;
  const int h = bh % f.H, b = bh / f.H;
  for (int i = threadIdx.x; i < 2 * 1024; i += blockDim.x) (&sh[0][0])[i] = 0;
  __syncthreads();
  const uint32_t q0 = sel[h * 8 + 0] >> 10, q1 = sel[h * 8 + 2] >> 10;
  const bool same = q0 == q1;
  const float thr_lo = __uint_as_float(band[h * kBandWords + 0]), thr_hi = __uint_as_float(band[h * kBandWords + 1]);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, l16 = lane & 15;
  int per = (f.T_new + gridDim.x - 1) / gridDim.x;
  per = (per + kF32Tok - 1) / kF32Tok * kF32Tok;
  const int t0 = blockIdx.x * per, t1 = min(f.T_new, t0 + per);
  const uint16_t* base = f.x + b * f.xs_b + h * f.xs_h + 8 * l16;
  const bool cb16 = ib + rbits == 16;
  const uint32_t rmask16 = (0xffffu >> ib) << ib;             // radius bits of a 16-bit field
  for (int tb = t0 + warp * 2; tb < t1; tb += kF32Tok) {      // warp-uniform trip count: the halves shuffle below
    const int t = tb + (lane >> 4);
    uint4 r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (t + 16 * u < t1) r[u] = *reinterpret_cast<const uint4*>(base + (int64_t)(t + 16 * u) * f.xs_t);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int tu = t + 16 * u;
      const bool live = tu < t1;
      uint32_t m = 0;
      if (live) {
        float n[2];
        norms_of_two<DT>(r[u], n[0], n[1]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t key = __float_as_uint(n[e]);
          const uint32_t top = key >> 10;
          if (top == q0) atomicAdd(&sh[0][key & 0x3ffu], 1u);
          else if (top == q1) atomicAdd(&sh[1][key & 0x3ffu], 1u);
          if (n[e] > thr_hi) m |= 1u << e;
          else if (n[e] > thr_lo) {
            const uint32_t pos = atomicAdd(&band[h * kBandWords + 2], 1u);
            const int c32 = 2 * l16 + e;
            if (pos < (uint32_t)kUndCap)
              und[(int64_t)h * kUndCap + pos] =
                  f.pair ? (uint32_t)(((int64_t)b * (2 * f.T_new) + 2 * tu + (c32 >> 4)) * 32 + (c32 & 15))
                         : (uint32_t)(((int64_t)b * f.T_new + tu) * 32 + c32);
          }
        }
      }
      // the token's flag word: OR of the 16 lanes that share it (bits 2*l16 and 2*l16 + 1 each)
      uint32_t word = m << (2 * l16);
      word |= __shfl_xor_sync(0xffffffffu, word, 1);
      word |= __shfl_xor_sync(0xffffffffu, word, 2);
      word |= __shfl_xor_sync(0xffffffffu, word, 4);
      word |= __shfl_xor_sync(0xffffffffu, word, 8);
      if (live) {
        const int64_t row = (int64_t)bh * dst.T_cap + t_start + (f.pair ? 2 * tu : tu);   // (pairs: two contiguous rows)
        if (m) {
          uint32_t* rowp = reinterpret_cast<uint32_t*>(dst.codes + row * dst.row_bytes);
          if (cb16) {
            // 16-bit fields: both chunks of this lane live in word l16 of the row, one atomic clears either or both
            atomicAnd(&rowp[l16], ~(((m & 1u) ? rmask16 : 0u) | ((m & 2u) ? rmask16 << 16 : 0u)));
          } else {
            if (m & 1u) clear_radius(rowp, 2 * l16, ib, rbits);
            if (m & 2u) clear_radius(rowp, 2 * l16 + 1, ib, rbits);
          }
        }
        if (l16 == 0) {
          if (f.pair) { dst.flags[row] = word & 0xffffu; dst.flags[row + 1] = word >> 16; }
          else dst.flags[row] = word;
        }
      }
    }
  }
  __syncthreads();
  uint32_t* gh = hist + ((int64_t)h * 3 + 2) * 2 * kHistBins;
  for (int i = threadIdx.x; i < 1024; i += blockDim.x) {
    const uint32_t c0 = sh[0][i], c1 = same ? c0 : sh[1][i];
    if (c0) atomicAdd(&gh[i], c0);
    if (c1) atomicAdd(&gh[kHistBins + i], c1);
  }
}

// The undecided chunks of one head against the exact threshold (one CTA per head).
template <int DT>
__global__ void __launch_bounds__(256)
fixup_list_kernel(Fast32 f, hqmq_packed dst, int t_start, int ib, int rbits, const uint32_t* __restrict__ sel,
                  const uint32_t* __restrict__ band, const uint32_t* __restrict__ und, const uint32_t* __restrict__ gate,
                  int gate_want, int und_cap) {
  if (gate && (*gate != 0u) != (gate_want != 0)) return;   // (this launch belongs to the other of the two paths)
  const int h = blockIdx.x;
  const uint32_t n = band[h * kBandWords + 2];
  if (n == 0 || n > (uint32_t)und_cap) return;
  const float thr = __uint_as_float(sel[h * 8 + 6]);
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
    const uint32_t e = und[(int64_t)h * und_cap + i];
    const int c = e & 31;
    const int64_t bt = e >> 5;
    const int b = (int)(bt / f.T_new), t = (int)(bt - (int64_t)b * f.T_new);
    const uint2 raw = *reinterpret_cast<const uint2*>(f.x + b * f.xs_b + h * f.xs_h + (int64_t)t * f.xs_t + 4 * c);
    float v[4];
    v[0] = bits16_to_float(raw.x & 0xffff, DT); v[1] = bits16_to_float(raw.x >> 16, DT);
    v[2] = bits16_to_float(raw.y & 0xffff, DT); v[3] = bits16_to_float(raw.y >> 16, DT);
    if (chunk_norm(v) > thr) flag_late(dst, ((int64_t)b * f.H + h) * dst.T_cap + t_start + t, c, ib, rbits);
  }
}

// Fallback when a head's list overflowed: re-read x and settle every chunk between the two bounds.
template <int DT>
__global__ void __launch_bounds__(256)
fixup_scan_kernel(Fast32 f, hqmq_packed dst, int t_start, int ib, int rbits, const uint32_t* __restrict__ sel,
                  const uint32_t* __restrict__ band, const uint32_t* __restrict__ gate, int gate_want, int und_cap) {
  if (gate && (*gate != 0u) != (gate_want != 0)) return;   // (this launch belongs to the other of the two paths)
  const int bh = blockIdx.y;
  const int h = bh % f.H, b = bh / f.H;
  if (band[h * kBandWords + 2] <= (uint32_t)und_cap) return;
  const float thr = __uint_as_float(sel[h * 8 + 6]);
  const float thr_lo = __uint_as_float(band[h * kBandWords + 0]), thr_hi = __uint_as_float(band[h * kBandWords + 1]);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, l16 = lane & 15;
  int per = (f.T_new + gridDim.x - 1) / gridDim.x;
  per = (per + kF32Tok - 1) / kF32Tok * kF32Tok;
  const int t0 = blockIdx.x * per, t1 = min(f.T_new, t0 + per);
  const uint16_t* base = f.x + b * f.xs_b + h * f.xs_h + 8 * l16;
  for (int t = t0 + warp * 2 + (lane >> 4); t < t1; t += 16) {
    const uint4 r = *reinterpret_cast<const uint4*>(base + (int64_t)t * f.xs_t);
    float n[2];
    norms_of_two<DT>(r, n[0], n[1]);
#pragma unroll
    for (int e = 0; e < 2; ++e)
      if (n[e] > thr_lo && !(n[e] > thr_hi) && n[e] > thr) {
        const int c32 = 2 * l16 + e;
        if (f.pair) flag_late(dst, (int64_t)bh * dst.T_cap + t_start + 2 * t + (c32 >> 4), c32 & 15, ib, rbits);
        else flag_late(dst, (int64_t)bh * dst.T_cap + t_start + t, c32, ib, rbits);
      }
  }
}

// Flags: one lane group per token.
__global__ void __launch_bounds__(256)
flags_kernel(EncGeom g, const void* __restrict__ x, hqmq_packed dst, int t_start, const uint32_t* __restrict__ sel) {
  const int bh = blockIdx.y;
  const int h = bh % g.H, b = bh / g.H;
  const float thr = __uint_as_float(sel[h * 8 + 6]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / g.npl, c = lane % g.npl;
  const int tok_per_iter = (blockDim.x >> 5) * g.tpw;
  for (int tb4 = blockIdx.x * tok_per_iter * 4; tb4 < g.T_new; tb4 += gridDim.x * tok_per_iter * 4) {
   float v4[4][4];
#pragma unroll
   for (int u = 0; u < 4; ++u) {   // four independent loads in flight per thread
     const int t = tb4 + u * tok_per_iter + warp * g.tpw + sub;
     v4[u][0] = v4[u][1] = v4[u][2] = v4[u][3] = 0.f;
     if (t < g.T_new && c < g.n) load_chunk(x, b * g.xs_b + h * g.xs_h + t * g.xs_t + 4 * c, g.x_dtype, v4[u]);
   }
#pragma unroll
   for (int u = 0; u < 4; ++u) {
    const int tb = tb4 + u * tok_per_iter;
    if (tb >= g.T_new) break;
    const int t = tb + warp * g.tpw + sub;
    const bool active = t < g.T_new && c < g.n;
    const float* v = v4[u];
    const bool f = active && chunk_norm(v) > thr;
    const uint32_t bal = __ballot_sync(0xffffffffu, f);
    if (f) {
      // A flagged chunk is stored in the side buffer: its radius code in the packed row becomes 0 so
      // that decoding the row contributes nothing for it.
      const int cb = g.ib + g.rbits;
      uint32_t* rowp = reinterpret_cast<uint32_t*>(dst.codes + ((int64_t)bh * dst.T_cap + t_start + t) * dst.row_bytes);
      const int lo = c * cb + g.ib, hi = (c + 1) * cb;   // bit range of the radius code
      const int w0 = lo >> 5, w1 = (hi - 1) >> 5;
      const uint32_t m0 = ~0u << (lo & 31);
      const uint32_t m1 = (hi & 31) ? ~(~0u << (hi & 31)) : ~0u;
      if (w0 == w1) atomicAnd(&rowp[w0], ~(m0 & m1));
      else { atomicAnd(&rowp[w0], ~m0); atomicAnd(&rowp[w1], ~m1); }
    }
    if (t < g.T_new && c == 0) {
      const uint32_t mask = g.npl == 32 ? 0xffffffffu : ((1u << g.npl) - 1u);
      const uint32_t word = (bal >> (sub * g.npl)) & mask;
      dst.flags[(int64_t)bh * dst.T_cap + t_start + t] = word;
    }
   }
  }
}

// Distinct flagged chunk positions of a 16-token block -> records the block owns (0 when it has none,
// or more than HQMQ_OFRAG_MAX_PER_TILE records would be needed).
__device__ __forceinline__ int ofrag_records_for(uint32_t any_c) {
  const int nd = __popc(any_c);
  const int ng = (nd + 3) >> 2;
  return ng <= HQMQ_OFRAG_MAX_PER_TILE ? ng : 0;
}

// Per (b,h), one CTA of 8 warps, one lane per 16-token block of this call: the block's flagged chunks are
// counted from its flag words and scanned into the payload offsets; with a fragment plane, also the record
// offsets (a block gets records in the call that completes it; a block whose records would pass the capacity,
// and every block after it in this call, gets none: the running total is monotone, so that is every block
// whose inclusive total exceeds the capacity).  `payload` = 0 on a call without Med3x (nothing flagged).
constexpr int kScanWarps = 8;
constexpr int kScanIters = 16;     // blocks per lane: up to 8 * 32 * 16 = 4096 blocks (64 k tokens) in one sweep
__device__ __forceinline__ void
scan_body(const hqmq_packed& dst, int t_start, int T_new, int blk0, int nblk, int payload, uint32_t* __restrict__ status) {
  __shared__ uint32_t w_tot[kScanWarps], w_ftot[kScanWarps], s_last_ok[kScanWarps];
  const int bh = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb_cap = dst.T_cap / HQMQ_OUT_BLOCK + 1;
  uint32_t* off = dst.out_off + (int64_t)bh * nb_cap;
  uint32_t* foff = dst.ofrag ? dst.ofrag_off + (int64_t)bh * nb_cap : nullptr;
  const uint32_t* fl = dst.flags + (int64_t)bh * dst.T_cap;
  uint32_t run = payload ? dst.out_count[bh] : 0u;
  uint32_t frun = foff ? foff[blk0] : 0u;
  const int t_end = t_start + T_new;
  const int sweep = kScanWarps * 32 * kScanIters;
  bool full = false;       // a block of an earlier sweep did not fit the record capacity
  for (int s0 = 0; s0 < nblk; s0 += sweep) {
    // warp w owns the contiguous blocks [s0 + w*32*kScanIters, ...): lane-major inside an iteration
    uint32_t c[kScanIters], fc[kScanIters];
    uint32_t wsum = 0, wfsum = 0;
#pragma unroll
    for (int it = 0; it < kScanIters; ++it) {
      const int i = s0 + (warp * kScanIters + it) * 32 + lane, ba = blk0 + i;
      uint32_t cc = 0, any_c = 0;
      // (an iteration whose 32 blocks all lie past the call -- every one but the first in a one-token append --
      //  is skipped here and in the scan below: it would add zeros)
      if (i - lane >= nblk) { c[it] = fc[it] = 0u; continue; }
      if (i < nblk) {
        const int tb = ba * HQMQ_OUT_BLOCK;
#pragma unroll
        for (int q = 0; q < HQMQ_OUT_BLOCK / 4; ++q) {
          const uint4 w = *reinterpret_cast<const uint4*>(fl + tb + 4 * q);
          const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int t = tb + 4 * q + k;
            if (t >= t_start && t < t_end) cc += __popc(ww[k]);   // payload entries: tokens of this call only
            if (t < t_end) any_c |= ww[k];                          // records: every token the block holds
          }
        }
      }
      // a block gets its records in the call that completes it (all 16 tokens present), from flags and payload
      const bool complete = i < nblk && (ba + 1) * HQMQ_OUT_BLOCK <= t_end;
      c[it] = cc;
      fc[it] = foff && complete ? (uint32_t)ofrag_records_for(any_c) : 0u;
      wsum += cc; wfsum += fc[it];
    }
    wsum = __reduce_add_sync(0xffffffffu, wsum);
    wfsum = __reduce_add_sync(0xffffffffu, wfsum);
    if (lane == 0) { w_tot[warp] = wsum; w_ftot[warp] = wfsum; }
    __syncthreads();
    uint32_t base = run, fbase = frun, all = 0, fall = 0;
    for (int w = 0; w < kScanWarps; ++w) {
      if (w < warp) { base += w_tot[w]; fbase += w_ftot[w]; }
      all += w_tot[w]; fall += w_ftot[w];
    }
    uint32_t my_last_ok = frun;      // largest inclusive record total within the capacity seen by this warp
#pragma unroll
    for (int it = 0; it < kScanIters; ++it) {
      const int i = s0 + (warp * kScanIters + it) * 32 + lane, ba = blk0 + i;
      if (i - lane >= nblk) continue;
      uint32_t incl = c[it], fincl = fc[it];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        const uint32_t fv = __shfl_up_sync(0xffffffffu, fincl, o);
        if (lane >= o) { incl += v; fincl += fv; }
      }
      if (payload) {
        // A block that already holds tokens from an earlier call keeps its offset.
        if (i < nblk && !(i == 0 && (t_start % HQMQ_OUT_BLOCK) != 0)) off[ba] = base + incl - c[it];
        base += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (foff) {
        fincl += fbase;
        const bool ok = !full && fincl <= (uint32_t)dst.ofrag_cap;
        fc[it] = ok ? fincl : 0xffffffffu;      // reused: the inclusive total, or "over the capacity"
        if (ok && i < nblk) my_last_ok = max(my_last_ok, fincl);
        fbase = __shfl_sync(0xffffffffu, fincl, 31);
      }
    }
    if (foff) {
      my_last_ok = __reduce_max_sync(0xffffffffu, my_last_ok);
      if (lane == 0) s_last_ok[warp] = my_last_ok;
      __syncthreads();
      uint32_t last_ok = frun;
      for (int w = 0; w < kScanWarps; ++w) last_ok = max(last_ok, s_last_ok[w]);
#pragma unroll
      for (int it = 0; it < kScanIters; ++it) {
        const int i = s0 + (warp * kScanIters + it) * 32 + lane;
        if (i < nblk) foff[blk0 + i + 1] = fc[it] != 0xffffffffu ? fc[it] : last_ok;
      }
      full = full || frun + fall > last_ok;   // some block of this sweep was over the capacity
      frun = last_ok;
    }
    run += all;
    __syncthreads();      // w_tot / s_last_ok are rewritten by the next sweep
  }
  if (payload && threadIdx.x == 0) {
    off[blk0 + nblk] = run;
    if (run > (uint32_t)dst.out_cap) atomicOr(&status[0], 1u);
    dst.out_count[bh] = run;
  }
}

__global__ void __launch_bounds__(kScanWarps * 32)
scan_kernel(hqmq_packed dst, int t_start, int T_new, int blk0, int nblk, int payload, uint32_t* __restrict__ status) {
  scan_body(dst, t_start, T_new, blk0, nblk, payload, status);
}

// Side planes of one 16-token block, one warp per block: the payload (original values of every flagged chunk,
// in (token, chunk) order) and, for a block that owns fragment records, the records (layout in
// include/hqmq_b200.h).  Lane l < 16 holds the flag word of token l of the block.
__device__ __forceinline__ void
side_block(const EncGeom& g, const void* __restrict__ x, const hqmq_packed& dst, int t_start, int blk0, int nblk, int bh, int i,
           int lane) {
  const int h = bh % g.H, b = bh / g.H;
  if (i >= nblk) return;
  const int ba = blk0 + i;
  const int nb_cap = dst.T_cap / HQMQ_OUT_BLOCK + 1;
  const int64_t row0 = (int64_t)bh * dst.T_cap + (int64_t)ba * HQMQ_OUT_BLOCK;
  const uint32_t fw = lane < HQMQ_OUT_BLOCK ? dst.flags[row0 + lane] : 0u;
  uint32_t any_c = __reduce_or_sync(0xffffffffu, fw);
  if (!any_c) return;
  const int64_t xbase = b * g.xs_b + h * g.xs_h;

  // ---- payload: lane pair (l, l + 16) shares token l; the pair takes the token's flagged chunks alternately ----
  uint32_t excl16;   // lanes 0..15: flagged chunks of the block's earlier tokens
  const uint32_t off0 = dst.out_off[(int64_t)bh * nb_cap + ba];
  const int esz = dst.out_dtype == HQMQ_F32 ? 4 : 2;
  unsigned char* base = reinterpret_cast<unsigned char*>(dst.out_vals) + (int64_t)bh * dst.out_cap * 4 * esz;
  {
    uint32_t incl = __popc(fw);
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
      if ((lane & 15) >= o) incl += v;
    }
    excl16 = incl - __popc(fw);
    const uint32_t before = __shfl_sync(0xffffffffu, excl16, lane & 15);
    uint32_t word = __shfl_sync(0xffffffffu, fw, lane & 15);
    const int t = ba * HQMQ_OUT_BLOCK + (lane & 15) - t_start;                         // token index within this call
    if (t >= 0 && t < g.T_new && word) {
      uint32_t pos = off0 + before;
      int k = 0;
      while (word) {
        const int c = __ffs(word) - 1;
        word &= word - 1;
        if ((k & 1) == (lane >> 4) && pos < (uint32_t)dst.out_cap) {
          float v[4];
          load_chunk(x, xbase + t * g.xs_t + 4 * c, g.x_dtype, v);
          if (dst.out_dtype == HQMQ_F32) {
            *reinterpret_cast<float4*>(base + (int64_t)pos * 16) = make_float4(v[0], v[1], v[2], v[3]);
          } else {
            uint2 o;
            o.x = float_to_bits16(v[0], dst.out_dtype) | ((uint32_t)float_to_bits16(v[1], dst.out_dtype) << 16);
            o.y = float_to_bits16(v[2], dst.out_dtype) | ((uint32_t)float_to_bits16(v[3], dst.out_dtype) << 16);
            *reinterpret_cast<uint2*>(base + (int64_t)pos * 8) = o;
          }
        }
        ++pos; ++k;
      }
    }
  }

  // ---- fragment records: built from the flags and the payload, so that a block filled by several calls
  // (token-by-token appends) gets them too, in the call that completes it -------------------------------------
  if (!dst.ofrag) return;
  const uint32_t* off = dst.ofrag_off + (int64_t)bh * nb_cap;
  const uint32_t o0 = off[ba], o1 = off[ba + 1];
  if (o1 <= o0) return;
  __threadfence_block();
  __syncwarp();            // this call's payload entries of the block were written by other lanes of the warp
  const int j = lane & 3, r = lane >> 2;
  uint32_t fl[2], pre[2]; float inv[2];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    fl[nt] = __shfl_sync(0xffffffffu, fw, nt * 8 + r);
    pre[nt] = __shfl_sync(0xffffffffu, excl16, nt * 8 + r);
    inv[nt] = fl[nt] ? (float)g.qmax / load_scale(dst, row0 + nt * 8 + r) : 0.f;
  }
  for (uint32_t rec = o0; rec < o1; ++rec) {
    int cj = -1;
    uint32_t hdr = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int c = any_c ? __ffs(any_c) - 1 : -1;
      any_c &= any_c - 1;
      if (q == j) cj = c;
      hdr |= (uint32_t)(c & 0xff) << (8 * q);
    }
    uint32_t a[4] = {0u, 0u, 0u, 0u};
    if (cj >= 0) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        if ((fl[nt] >> cj) & 1u) {
          const uint32_t pos = off0 + pre[nt] + __popc(fl[nt] & ((1u << cj) - 1u));
          float v[4] = {0.f, 0.f, 0.f, 0.f};
          if (pos < (uint32_t)dst.out_cap) {     // (an entry dropped by an overflowing side buffer reads as 0)
            if (dst.out_dtype == HQMQ_F32) {
              const float4 f = *reinterpret_cast<const float4*>(base + (int64_t)pos * 16);
              v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            } else {
              const uint2 o = *reinterpret_cast<const uint2*>(base + (int64_t)pos * 8);
              v[0] = bits16_to_float(o.x & 0xffff, dst.out_dtype); v[1] = bits16_to_float(o.x >> 16, dst.out_dtype);
              v[2] = bits16_to_float(o.y & 0xffff, dst.out_dtype); v[3] = bits16_to_float(o.y >> 16, dst.out_dtype);
            }
          }
          const __half2 h01 = __floats2half2_rn(v[0] * inv[nt], v[1] * inv[nt]);
          const __half2 h23 = __floats2half2_rn(v[2] * inv[nt], v[3] * inv[nt]);
          a[nt] = *reinterpret_cast<const uint32_t*>(&h01);
          a[2 + nt] = *reinterpret_cast<const uint32_t*>(&h23);
        }
      }
    }
    unsigned char* recp = dst.ofrag + ((int64_t)bh * dst.ofrag_cap + rec) * HQMQ_OFRAG_BYTES;
    if (lane == 0) *reinterpret_cast<uint4*>(recp) = make_uint4(hdr, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(recp + 16 + lane * 16) = make_uint4(a[0], a[1], a[2], a[3]);
  }
}

// (grid (blocks / warps per CTA, B * H): one warp per block)
__device__ __forceinline__ void
side_body(const EncGeom& g, const void* __restrict__ x, const hqmq_packed& dst, int t_start, int blk0, int nblk) {
  side_block(g, x, dst, t_start, blk0, nblk, blockIdx.y, blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), threadIdx.x & 31);
}
__global__ void __launch_bounds__(256)
side_kernel(EncGeom g, const void* __restrict__ x, hqmq_packed dst, int t_start, int blk0, int nblk) {
  side_body(g, x, dst, t_start, blk0, nblk);
}

// The offset scan of scan_body for a call that touches at most 32 blocks of a (b, h): one warp, one lane per block, a
// single sweep.  Same results word for word (payload offsets of the blocks this call starts, record offsets of the
// blocks it completes with the capacity rule, the running totals).
constexpr int kScanSmallBlocks = 32;
__device__ __forceinline__ void
scan_small_warp(const hqmq_packed& dst, int bh, int t_start, int T_new, int blk0, int nblk, int payload,
                uint32_t* __restrict__ status, int lane) {
  const int nb_cap = dst.T_cap / HQMQ_OUT_BLOCK + 1;
  uint32_t* off = dst.out_off + (int64_t)bh * nb_cap;
  uint32_t* foff = dst.ofrag ? dst.ofrag_off + (int64_t)bh * nb_cap : nullptr;
  const uint32_t* fl = dst.flags + (int64_t)bh * dst.T_cap;
  // (the totals are read by one lane and handed round, so that the reads are done before lane 0 rewrites them)
  uint32_t run = 0u, frun = 0u;
  if (lane == 0) { run = payload ? dst.out_count[bh] : 0u; frun = foff ? foff[blk0] : 0u; }
  run = __shfl_sync(0xffffffffu, run, 0);
  frun = __shfl_sync(0xffffffffu, frun, 0);
  const int t_end = t_start + T_new;
  const int i = lane, ba = blk0 + i;
  uint32_t cc = 0, any_c = 0;
  if (i < nblk) {
    const int tb = ba * HQMQ_OUT_BLOCK;
#pragma unroll
    for (int q = 0; q < HQMQ_OUT_BLOCK / 4; ++q) {
      const uint4 w = *reinterpret_cast<const uint4*>(fl + tb + 4 * q);
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int t = tb + 4 * q + k;
        if (t >= t_start && t < t_end) cc += __popc(ww[k]);
        if (t < t_end) any_c |= ww[k];
      }
    }
  }
  const bool complete = i < nblk && (ba + 1) * HQMQ_OUT_BLOCK <= t_end;
  const uint32_t fcnt = foff && complete ? (uint32_t)ofrag_records_for(any_c) : 0u;
  uint32_t incl = cc, fincl = fcnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    const uint32_t fv = __shfl_up_sync(0xffffffffu, fincl, o);
    if (lane >= o) { incl += v; fincl += fv; }
  }
  if (payload && i < nblk && !(i == 0 && (t_start % HQMQ_OUT_BLOCK) != 0)) off[ba] = run + incl - cc;
  if (foff) {
    fincl += frun;
    const bool ok = fincl <= (uint32_t)dst.ofrag_cap;
    const uint32_t last_ok = __reduce_max_sync(0xffffffffu, ok && i < nblk ? fincl : frun);
    if (i < nblk) foff[ba + 1] = ok ? fincl : last_ok;
  }
  const uint32_t total = run + __shfl_sync(0xffffffffu, incl, 31);
  if (payload && lane == 0) {
    off[blk0 + nblk] = total;
    if (total > (uint32_t)dst.out_cap) atomicOr(&status[0], 1u);
    dst.out_count[bh] = total;
  }
}

// The K + V append of a layer in ONE launch, grid (H, 2): blockIdx.y = 0 the K tensor, 1 the V tensor (same batch,
// heads, tokens and head dim).  After the head's codes, scales and flags, the same CTA scans the offsets of its batch
// entries (a warp per entry) and writes their side planes (a warp per block) -- what scan_kernel and side_kernel do in
// two more launches of a single-tensor call.  For calls that touch at most kScanSmallBlocks blocks per (b, h).
// The status words are cleared by the host (a memset ahead of the launch): a CTA may report an overflow before
// another CTA has started.
__global__ void __launch_bounds__(kSmallThreads) append_pair_kernel(SmallPair p) {
  const SmallArgs& a = p.t[blockIdx.y];
  encode_small_body(a.g, a.x, a.qs, a.dst, a.t_start, p.maps, a.joint, a.lut, a.nmul, a.C, a.med_out, a.quantile);
  if (!a.scan) return;
  __syncthreads();          // the head's flag words and scales are in global memory for the other warps of the CTA
  const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int b = warp; b < a.g.B; b += kSmallThreads / 32)
    scan_small_warp(a.dst, b * a.g.H + h, a.t_start, a.g.T_new, a.blk0, a.nblk, a.payload, a.status, lane);
  if (!a.side) return;
  __syncthreads();          // ... and so are the offsets
  for (int w = warp; w < a.g.B * a.nblk; w += kSmallThreads / 32) {
    const int b = w / a.nblk, i = w - b * a.nblk;
    side_block(a.g, a.x, a.dst, a.t_start, a.blk0, a.nblk, b * a.g.H + h, i, lane);
  }
}

// ---- look-up table construction ---------------------------------------------------------------------
// Geometry (the same for every head): per (cx, cy) column the stored cz range = the cells whose grown box meets
// the octahedron |w1| + |w2| + |w3| <= 1, and the index of the column's first cell.
__device__ __forceinline__ float min_abs_over(float lo, float hi) { return (lo <= 0.f && hi >= 0.f) ? 0.f : fminf(fabsf(lo), fabsf(hi)); }
__global__ void __launch_bounds__(1024) lut_rows_kernel(int n, uint32_t* __restrict__ ghdr, uint32_t* __restrict__ rows) {
  __shared__ uint32_t s_cnt[kLutRows], s_min[kLutRows];
  const float step = 2.0f / (float)n;
  for (int col = threadIdx.x; col < n * n; col += blockDim.x) {
    const int cx = col / n, cy = col - cx * n;
    const float m1 = min_abs_over(cx * step - 1.f - kLutBoxEps, (cx + 1) * step - 1.f + kLutBoxEps);
    const float m2 = min_abs_over(cy * step - 1.f - kLutBoxEps, (cy + 1) * step - 1.f + kLutBoxEps);
    const float lim = 1.f + kLutBoxEps - m1 - m2;
    int zmin = n, zmax = -1;
    for (int cz = 0; cz < n; ++cz) {
      const float m3 = min_abs_over(cz * step - 1.f - kLutBoxEps, (cz + 1) * step - 1.f + kLutBoxEps);
      if (m3 <= lim) { zmin = min(zmin, cz); zmax = max(zmax, cz); }
    }
    s_cnt[col] = zmax >= zmin ? (uint32_t)(zmax - zmin + 1) : 0u;
    s_min[col] = zmax >= zmin ? (uint32_t)zmin : 0u;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t run = 0;
    for (int col = 0; col < n * n; ++col) {
      rows[col] = run | (s_min[col] << 20) | (s_cnt[col] << 26);
      run += s_cnt[col];
    }
    ghdr[0] = (uint32_t)n; ghdr[1] = run; ghdr[2] = ghdr[3] = 0u;
  }
}

// One CTA per ((cx, cy) column, head), walking the column's stored cells.  tmp: [H][kLutCellCap][kLutMaxList] uint16
// candidate lists (ascending), cnt: [H][kLutCellCap] list lengths (0 = too long: exhaustive search in that cell).
__global__ void __launch_bounds__(128)
lut_cells_kernel(const float* __restrict__ joint_all, int S, int n, const uint32_t* __restrict__ rows,
                 uint16_t* __restrict__ tmp, uint32_t* __restrict__ cnt) {
  __shared__ float s_best[4];
  __shared__ int s_bk[4];
  __shared__ int s_n;
  __shared__ uint16_t s_list[kLutMaxList];
  __shared__ float4 s_cw[kLutMaxList];
  __shared__ unsigned char s_drop[kLutMaxList];
  const int col = blockIdx.x, h = blockIdx.y, K = 24 * S;
  const float4* joint = reinterpret_cast<const float4*>(joint_all) + (int64_t)h * K;
  const uint32_t row = rows[col];
  const int zcnt = (int)(row >> 26), zmin = (int)((row >> 20) & 63u), base = (int)(row & 0xfffffu);
  const int cx = col / n, cy = col - cx * n;
  const float step = 2.0f / (float)n;
  const float w1 = (cx + 0.5f) * step - 1.f, w2 = (cy + 0.5f) * step - 1.f;
  const float hh = 0.5f * step + kLutBoxEps;
  for (int zc = 0; zc < zcnt; ++zc) {
    const int cell = base + zc;
    const float w3 = (zmin + zc + 0.5f) * step - 1.f;
    // winner at the centre of the cell
    float best = -1e30f; int bk = 0;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      const float4 c = joint[k];
      const float sim = c.x + w1 * c.y + w2 * c.z + w3 * c.w;
      if (sim > best) { best = sim; bk = k; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int ok = __shfl_xor_sync(0xffffffffu, bk, o);
      if (ob > best || (ob == best && ok < bk)) { best = ob; bk = ok; }
    }
    if ((threadIdx.x & 31) == 0) { s_best[threadIdx.x >> 5] = best; s_bk[threadIdx.x >> 5] = bk; }
    if (threadIdx.x == 0) s_n = 0;
    __syncthreads();
    best = s_best[0]; bk = s_bk[0];
    for (int i = 1; i < 4; ++i)
      if (s_best[i] > best || (s_best[i] == best && s_bk[i] < bk)) { best = s_best[i]; bk = s_bk[i]; }
    const float4 cs = joint[bk];
    // every codeword that is not beaten by the centre's winner over the whole (grown) box
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      const float4 c = joint[k];
      const float d0 = c.x - cs.x, d1 = c.y - cs.y, d2 = c.z - cs.z, d3 = c.w - cs.w;
      const float ub = d0 + d1 * w1 + d2 * w2 + d3 * w3 + hh * (fabsf(d1) + fabsf(d2) + fabsf(d3));
      if (ub >= -kLutMargin) {
        const int pos = atomicAdd(&s_n, 1);
        if (pos < kLutMaxList) s_list[pos] = (uint16_t)k;
      }
    }
    __syncthreads();
    int m = s_n;
    if (m > kLutMaxList) m = 0;         // too long: this cell falls back to the exhaustive search
    if (threadIdx.x == 0) {
      for (int i = 1; i < m; ++i) {     // ascending order makes the table reproducible
        const uint16_t v = s_list[i];
        int q = i - 1;
        while (q >= 0 && s_list[q] > v) { s_list[q + 1] = s_list[q]; --q; }
        s_list[q + 1] = v;
      }
    }
    __syncthreads();
    if (threadIdx.x < m) s_cw[threadIdx.x] = joint[s_list[threadIdx.x]];
    __syncthreads();
    // second filter: drop a codeword that loses to some OTHER listed codeword over the whole box
    if (threadIdx.x < m) {
      const float4 ci = s_cw[threadIdx.x];
      bool drop = false;
      for (int q = 0; q < m && !drop; ++q) {
        if (q == threadIdx.x) continue;
        const float4 cq = s_cw[q];
        const float d0 = ci.x - cq.x, d1 = ci.y - cq.y, d2 = ci.z - cq.z, d3 = ci.w - cq.w;
        const float ub = d0 + d1 * w1 + d2 * w2 + d3 * w3 + hh * (fabsf(d1) + fabsf(d2) + fabsf(d3));
        drop = ub < -kLutMargin;
      }
      s_drop[threadIdx.x] = drop ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint16_t* dst = tmp + ((int64_t)h * kLutCellCap + cell) * kLutMaxList;
      int q = 0;
      for (int i = 0; i < m; ++i)
        if (!s_drop[i]) dst[q++] = s_list[i];
      cnt[(int64_t)h * kLutCellCap + cell] = (uint32_t)q;
    }
    __syncthreads();
  }
}

// Per head: cell words and the padded candidate lists.  A list of one needs no entry; longer ones are padded to a
// multiple of four with their last codeword, and the first entry of a list's last group carries bit 15.
__global__ void __launch_bounds__(1024)
lut_pack_kernel(const uint16_t* __restrict__ tmp, const uint32_t* __restrict__ cnt, unsigned char* __restrict__ lut, int S) {
  __shared__ uint32_t s_sum[1024];
  const int h = blockIdx.x;
  const uint32_t* gh = reinterpret_cast<const uint32_t*>(lut);
  const int n_cells = (int)gh[1];
  unsigned char* head = lut + kLutOffHeads + (size_t)h * kLutHeadBytes;
  uint16_t* cells = reinterpret_cast<uint16_t*>(head + 16);
  uint16_t* cands = reinterpret_cast<uint16_t*>(head + 16 + (size_t)kLutCellCap * 2);
  const int per = (n_cells + 1023) / 1024;
  const int c0 = threadIdx.x * per, c1 = min(n_cells, c0 + per);
  uint32_t tot = 0;
  for (int c = c0; c < c1; ++c) {
    const uint32_t m = cnt[(int64_t)h * kLutCellCap + c];
    tot += m > 1 ? (m + 3u) & ~3u : 0u;
  }
  s_sum[threadIdx.x] = tot;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const uint32_t v = threadIdx.x >= o ? s_sum[threadIdx.x - o] : 0;
    __syncthreads();
    s_sum[threadIdx.x] += v;
    __syncthreads();
  }
  const uint32_t total = s_sum[1023];
  const bool valid = total <= (uint32_t)kLutCandCap && n_cells <= kLutCellCap && 24 * S < 32768;
  if (threadIdx.x == 0) {
    uint32_t* hh = reinterpret_cast<uint32_t*>(head);
    hh[0] = valid ? total : 0u; hh[1] = valid ? 1u : 0u; hh[2] = hh[3] = 0u;
  }
  if (!valid) return;
  uint32_t run = s_sum[threadIdx.x] - tot;
  for (int c = c0; c < c1; ++c) {
    const uint32_t m = cnt[(int64_t)h * kLutCellCap + c];
    const uint16_t* src = tmp + ((int64_t)h * kLutCellCap + c) * kLutMaxList;
    if (m == 0) cells[c] = 0xffffu;
    else if (m == 1) cells[c] = (uint16_t)(0x8000u | src[0]);
    else {
      const uint32_t pm = (m + 3u) & ~3u;
      cells[c] = (uint16_t)(run >> 2);
      for (uint32_t i = 0; i < pm; ++i) {
        uint16_t v = src[i < m ? i : m - 1];
        if (i == pm - 4) v |= 0x8000u;
        cands[run + i] = v;
      }
      run += pm;
    }
  }
}

// (unit g) * (primary p) for all 24 units, as the native primary code (a << 3) | u of the product
Mul24 make_mul24_native() {
  auto prim = [](int p, double v[4]) {
    for (int i = 0; i < 4; ++i) v[i] = 0;
    if (p < 8) v[p >> 1] = (p & 1) ? -1.0 : 1.0;
    else for (int i = 0; i < 4; ++i) v[i] = (((p - 8) >> (3 - i)) & 1) ? -0.5 : 0.5;
  };
  Mul24 m;
  for (int g = 0; g < 24; ++g)
    for (int p = 0; p < 24; ++p) {
      double a[4], b[4], c[4];
      prim(g, a); prim(p, b);
      c[0] = a[0] * b[0] - a[1] * b[1] - a[2] * b[2] - a[3] * b[3];
      c[1] = a[0] * b[1] + a[1] * b[0] + a[2] * b[3] - a[3] * b[2];
      c[2] = a[0] * b[2] - a[1] * b[3] + a[2] * b[0] + a[3] * b[1];
      c[3] = a[0] * b[3] + a[1] * b[2] - a[2] * b[1] + a[3] * b[0];
      int ref = 0;
      for (int q = 0; q < 24; ++q) {
        double e[4];
        prim(q, e);
        double dd = 0;
        for (int i = 0; i < 4; ++i) dd += (e[i] - c[i]) * (e[i] - c[i]);
        if (dd < 1e-12) ref = q;
      }
      m.v[g][p] = index_maps().ref_to_native[ref];
    }
  return m;
}
const Mul24& mul24_native() {
  static const Mul24 m = make_mul24_native();
  return m;
}

inline size_t lut_bytes(int H) { return kLutOffHeads + (size_t)H * kLutHeadBytes + 576; }   // (+ the index table for small calls)
inline size_t lut_ws_bytes(int H) { return (size_t)H * kLutCellCap * 4 + (size_t)H * kLutCellCap * kLutMaxList * 2; }
// shared memory a main-pass kernel can give to a table next to its other arrays (fp32 joint table, histograms, rows)
inline size_t lut_smem_budget(int S) { return (size_t)226 * 1024 - (size_t)24 * S * 16 - (size_t)S * 16 - 3 * kHistBins * 4 - 4096; }

// Geometry of the main pass for the common case (d_head 128, 16-bit input): tokens per CTA and CTAs per (b, h).
struct MainGrid { int iters, gx; };
static MainGrid main_grid(int T_new, int B, int H) {
  MainGrid m;
  // tokens per CTA: long enough to amortise loading the tables, short enough to fill the machine twice
  int64_t it = ((int64_t)T_new * B * H + (int64_t)2 * 148 * kEnc32Warps - 1) / ((int64_t)2 * 148 * kEnc32Warps);
  m.iters = it < 1 ? 1 : it > 128 ? 128 : (int)it;
  m.gx = (T_new + kEnc32Warps * m.iters - 1) / (kEnc32Warps * m.iters);
  return m;
}
// The bracket pass pays when the sample predicts well: the statistic's sampling error falls with the square root of
// the sampled norms per head (a 1/32 sample of B * T_new tokens, 32 norms each), so the bracket's half-width is
// 3 / sqrt(norms) (about six standard errors of a median), at least 0.2 % and at most 1.2 %; calls too small for that,
// and quantiles out in the tails (few norms nearby: a much larger error), take the multi-pass path as before.
// d_head 64 as pairs of tokens (see EncGeom::pair16): the call's geometry must allow it.
static bool pair16_of(const hqmq_encode_args& a) {
  return a.dst.n_chunks == 16 && is_half_dtype(a.x_dtype) && a.x_stride[2] == 64 && a.T_new >= 2 && a.T_new % 2 == 0 &&
         a.t_start % 2 == 0;
}
constexpr int64_t kBracketMinTokens = 65536;     // B * T_new per head (of 32 chunks each)
static bool bracket_wanted(const hqmq_encode_args& a) {
  const bool pair = pair16_of(a);
  const int T32 = pair ? a.T_new / 2 : a.T_new;
  return a.median_mult > 0.f && !a.med_in && (a.dst.n_chunks == 32 || pair) && is_half_dtype(a.x_dtype) &&
         (int64_t)a.dst.B * T32 >= kBracketMinTokens && T32 >= 1024 &&
         (a.quantile == 0.f || (a.quantile >= 0.25f && a.quantile <= 0.75f));
}

struct WsPlan {
  size_t status, hist, sel, band, und, hist_s, sel_s, hist_fb, gate, bp, histA, histB, band_b, und_b, sel_b, rcnt, rlist, zero_bytes, total;
  int blk0, nblk, rcap, regions, und_cap;
};
WsPlan plan_ws(const hqmq_encode_args& a) {
  WsPlan w;
  const int H = a.dst.H;
  w.blk0 = a.t_start / HQMQ_OUT_BLOCK;
  w.nblk = a.T_new > 0 ? (a.t_start + a.T_new - 1) / HQMQ_OUT_BLOCK - w.blk0 + 1 : 0;
  size_t o = 0;
  w.status = o; o += 4;
  w.hist = o; o += (size_t)H * 3 * 2 * kHistBins;
  w.sel = o; o += (size_t)H * 8;
  w.band = o; o += (size_t)H * kBandWords;
  w.und = o; o += (size_t)H * kUndCap;
  w.hist_s = o; o += (size_t)H * 3 * 2 * kHistBins;   // sampled histograms (level-0 slot used)
  w.sel_s = o; o += (size_t)H * 8;
  w.hist_fb = o; o += (size_t)H * 2 * kHistBins;      // level 1 when the sample mispredicted
  // bracket mode of the main pass (reserved whenever the call could take it)
  w.gate = w.bp = w.histA = w.histB = w.band_b = w.und_b = w.sel_b = w.rcnt = w.rlist = 0;
  w.rcap = w.regions = w.und_cap = 0;
  w.zero_bytes = o * sizeof(uint32_t);
  if (bracket_wanted(a)) {
    const int T32 = pair16_of(a) ? a.T_new / 2 : a.T_new;
    const MainGrid mg = main_grid(T32, a.dst.B, H);
    w.regions = mg.gx * a.dst.B * H;
    w.rcap = kEnc32Warps * mg.iters * 32 / 16;        // a sixteenth of a CTA's chunks (the range holds about 2 %)
    w.gate = o; o += 4;
    w.bp = o; o += (size_t)H * kBpWords;
    w.histA = o; o += (size_t)H * kHistBins;
    w.histB = o; o += (size_t)H * 2 * kHistBins;
    w.band_b = o; o += (size_t)H * kBandWords;
    w.sel_b = o; o += (size_t)H * 8;
    w.rcnt = o; o += (size_t)w.regions;
    w.zero_bytes = o * sizeof(uint32_t);              // everything up to here starts at zero; the lists need not
    // the undecided list: the bracket is wider than the multi-pass path's band (a few per mille of the chunks of a
    // head with many outliers fall inside it)
    const int64_t per_head = (int64_t)a.dst.B * T32 * 32;
    w.und_cap = (int)(per_head / 256 > kUndCap ? (per_head / 256 < (1 << 20) ? per_head / 256 : (1 << 20)) : kUndCap);
    w.und_b = o; o += (size_t)H * w.und_cap;
    w.rlist = o; o += (size_t)w.regions * w.rcap;
  }
  w.total = o * sizeof(uint32_t);
  return w;
}

}  // namespace

}  // namespace hqmq

using namespace hqmq;

static int validate_encode(const hqmq_encode_args* a) {
  if (!a || a->struct_size != sizeof(hqmq_encode_args)) return HQMQ_ERR_ARG;
  if ((!a->x && a->T_new != 0) || !a->qs || !a->joint) return HQMQ_ERR_ARG;   // an empty input has no address
  if (!is_float_dtype(a->x_dtype)) return HQMQ_ERR_DTYPE;
  const bool med = a->median_mult > 0.f;
  int rc = check_packed(a->dst, med);
  if (rc) return rc;
  if (a->T_new < 0 || a->t_start < 0) return HQMQ_ERR_SHAPE;
  if (!(a->quantile >= 0.f && a->quantile < 1.f)) return HQMQ_ERR_ARG;
  if ((int64_t)a->t_start + a->T_new > a->dst.T_cap) return HQMQ_ERR_CAPACITY;
  const int align = a->x_dtype == HQMQ_F32 ? 16 : 8;
  if ((uintptr_t)a->x & (align - 1)) return HQMQ_ERR_ALIGN;
  for (int i = 0; i < 3; ++i)
    if (a->x_stride[i] % 4) return HQMQ_ERR_ALIGN;
  if (((uintptr_t)a->qs & 15) || ((uintptr_t)a->joint & 15)) return HQMQ_ERR_ALIGN;
  return HQMQ_OK;
}

extern "C" size_t hqmq_encode_lut_bytes(int H, int S) {
  if (H < 1 || S < 1 || 24 * S > 65536) return 0;
  return lut_bytes(H);
}
extern "C" size_t hqmq_encode_lut_workspace_bytes(int H, int S) {
  if (H < 1 || S < 1 || 24 * S > 65536) return 0;
  return lut_ws_bytes(H);
}
// Largest per-head candidate total of a built table, its grid, and whether every head is valid (synchronises).
static int lut_read(const void* lut, int H, cudaStream_t st, int& n, int& n_cells, int& max_total, bool& valid) {
  uint32_t gh[4];
  HQMQ_CHECK_CUDA(cudaMemcpyAsync(gh, lut, 16, cudaMemcpyDeviceToHost, st));
  HQMQ_CHECK_CUDA(cudaStreamSynchronize(st));
  n = (int)gh[0]; n_cells = (int)gh[1];
  max_total = 0; valid = n >= 2 && n <= kLutNMax && n_cells <= kLutCellCap;
  for (int h = 0; h < H && valid; ++h) {
    uint32_t v[2];
    HQMQ_CHECK_CUDA(cudaMemcpyAsync(v, reinterpret_cast<const unsigned char*>(lut) + kLutOffHeads + (size_t)h * kLutHeadBytes, 8,
                                    cudaMemcpyDeviceToHost, st));
    HQMQ_CHECK_CUDA(cudaStreamSynchronize(st));
    if (v[1] != 1u) valid = false;
    if ((int)v[0] > max_total) max_total = (int)v[0];
  }
  return HQMQ_OK;
}
extern "C" int hqmq_encode_lut_build(const float* joint, int H, int S, void* lut, size_t lut_nbytes, void* workspace,
                                     size_t ws_nbytes, void* stream) {
  if (!joint || !lut || !workspace) return HQMQ_ERR_ARG;
  if (H < 1 || S < 1 || 24 * S > 65536) return HQMQ_ERR_SHAPE;
  if (lut_nbytes < lut_bytes(H) || ws_nbytes < lut_ws_bytes(H)) return HQMQ_ERR_WORKSPACE;
  if (((uintptr_t)joint & 15) || ((uintptr_t)lut & 15) || ((uintptr_t)workspace & 15)) return HQMQ_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* L = reinterpret_cast<unsigned char*>(lut);
  uint32_t* cnt = reinterpret_cast<uint32_t*>(workspace);
  uint16_t* tmp = reinterpret_cast<uint16_t*>(cnt + (size_t)H * kLutCellCap);
  // the index table of the fold units, for the kernels that read the table in place
  HQMQ_CHECK_CUDA(cudaMemcpyAsync(L + kLutOffHeads + (size_t)H * kLutHeadBytes, &mul24_native(), 576, cudaMemcpyHostToDevice, st));
  // the finest grid whose tables fit the encoder's shared memory next to this codebook
  for (int n = kLutNMax; n >= 16; n -= 4) {
    lut_rows_kernel<<<1, 1024, 0, st>>>(n, reinterpret_cast<uint32_t*>(L), reinterpret_cast<uint32_t*>(L + kLutOffRows));
    lut_cells_kernel<<<dim3(n * n, H), 128, 0, st>>>(joint, S, n, reinterpret_cast<const uint32_t*>(L + kLutOffRows), tmp, cnt);
    lut_pack_kernel<<<H, 1024, 0, st>>>(tmp, cnt, L, S);
    HQMQ_LAUNCH_CHECK();
    int nn, n_cells, max_total; bool valid;
    const int rc = lut_read(lut, H, st, nn, n_cells, max_total, valid);
    if (rc) return rc;
    if (valid && lut_smem_bytes(nn, n_cells, max_total) <= lut_smem_budget(S)) return HQMQ_OK;
    if (24 * S >= 32768) break;          // codeword ids need 15 bits: no table for this codebook
  }
  // no grid fits: mark every head invalid (the encoder then searches exhaustively)
  for (int h = 0; h < H; ++h) HQMQ_CHECK_CUDA(cudaMemsetAsync(L + kLutOffHeads + (size_t)h * kLutHeadBytes, 0, 16, st));
  return HQMQ_OK;
}
extern "C" int hqmq_encode_lut_footprint(const void* lut, int H, int* footprint, void* stream) {
  if (!lut || !footprint || H < 1) return HQMQ_ERR_ARG;
  int n, n_cells, max_total; bool valid;
  const int rc = lut_read(lut, H, (cudaStream_t)stream, n, n_cells, max_total, valid);
  if (rc) return rc;
  *footprint = valid ? (int)lut_smem_bytes(n, n_cells, max_total) : -1;
  return HQMQ_OK;
}

// ---- Med3x median of a head whose batch entries live on several GPUs ---------------------------------------
// State: [H][3 levels][2 queries][kHistBins] histograms, then [H][8] select words (the layout select_kernel uses).
namespace hqmq {
namespace {
inline size_t med3x_state_words(int H) { return (size_t)H * 3 * 2 * kHistBins + (size_t)H * 8; }

__global__ void thr_from_median_kernel(const float* __restrict__ med_in, float C, int H, uint32_t* __restrict__ sel,
                                       float* __restrict__ med_out) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  const float med = med_in[h];
  sel[h * 8 + 6] = __float_as_uint(__fmul_rn(med, C));   // thr = med * C in fp32, like the local select
  sel[h * 8 + 7] = __float_as_uint(med);
  if (med_out) med_out[h] = med;
}
}  // namespace
}  // namespace hqmq
using namespace hqmq;

extern "C" size_t hqmq_med3x_state_bytes(int H) { return H < 1 ? 0 : med3x_state_words(H) * 4; }

extern "C" int hqmq_med3x_hist(const hqmq_encode_args* a, int level, void* state, size_t state_bytes, void* stream) {
  int rc = validate_encode(a);
  if (rc) return rc;
  if (level < 0 || level > 2) return HQMQ_ERR_ARG;
  const hqmq_packed& d = a->dst;
  if (!state || state_bytes < med3x_state_words(d.H) * 4) return HQMQ_ERR_WORKSPACE;
  if ((uintptr_t)state & 15) return HQMQ_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  uint32_t* hist = reinterpret_cast<uint32_t*>(state);
  uint32_t* sel = hist + (size_t)d.H * 3 * 2 * kHistBins;
  if (level == 0) HQMQ_CHECK_CUDA(cudaMemsetAsync(state, 0, med3x_state_words(d.H) * 4, st));
  if (a->T_new == 0) return HQMQ_OK;     // this GPU holds none of the head's tokens: its histograms stay zero
  EncGeom g;
  g.B = d.B; g.H = d.H; g.T_new = a->T_new; g.n = d.n_chunks;
  g.npl = 1; while (g.npl < g.n) g.npl <<= 1;
  g.tpw = 32 / g.npl;
  g.S = d.S; g.ib = idx_bits_for(d.S); g.rbits = d.radius_bits; g.qmax = (1 << d.radius_bits) - 1;
  g.x_dtype = a->x_dtype;
  g.xs_b = a->x_stride[0]; g.xs_h = a->x_stride[1]; g.xs_t = a->x_stride[2];
  const int bh_count = d.B * d.H;
  const int64_t per_bh = (int64_t)a->T_new * d.n_chunks;
  int hb = (148 * 16 + bh_count - 1) / bh_count;
  const int hb_max = (int)((per_bh + 256 * 16 - 1) / (256 * 16));
  if (hb > hb_max) hb = hb_max;
  if (hb < 1) hb = 1;
  hist_kernel<<<dim3(hb, bh_count), 256, 0, st>>>(g, a->x, hist, sel, level);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

extern "C" int hqmq_med3x_select(int H, int level, uint64_t n_total, float median_mult, void* state, size_t state_bytes,
                                 float* med_out, void* stream) {
  if (H < 1 || level < 0 || level > 2 || n_total < 1 || !(median_mult > 0.f)) return HQMQ_ERR_ARG;
  if (!state || state_bytes < med3x_state_words(H) * 4) return HQMQ_ERR_WORKSPACE;
  if ((uintptr_t)state & 15) return HQMQ_ERR_ALIGN;
  uint32_t* hist = reinterpret_cast<uint32_t*>(state);
  uint32_t* sel = hist + (size_t)H * 3 * 2 * kHistBins;
  select_kernel<<<H, 256, 0, (cudaStream_t)stream>>>(hist, sel, level, n_total, median_mult, level == 2 ? med_out : nullptr,
                                                     nullptr, nullptr, nullptr, 0.f, nullptr, 0);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

extern "C" size_t hqmq_encode_workspace_bytes(const hqmq_encode_args* a) {
  if (validate_encode(a) != HQMQ_OK) return 0;
  return plan_ws(*a).total;
}

static EncGeom geom_of(const hqmq_encode_args* a) {
  const hqmq_packed& d = a->dst;
  EncGeom g;
  g.B = d.B; g.H = d.H; g.T_new = a->T_new; g.n = d.n_chunks;
  g.npl = 1; while (g.npl < g.n) g.npl <<= 1;
  g.tpw = 32 / g.npl;
  g.S = d.S; g.ib = idx_bits_for(d.S); g.rbits = d.radius_bits; g.qmax = (1 << d.radius_bits) - 1;
  g.x_dtype = a->x_dtype;
  g.xs_b = a->x_stride[0]; g.xs_h = a->x_stride[1]; g.xs_t = a->x_stride[2];
  g.pair16 = 0;
  return g;
}

// Small calls (decode-time appends): one kernel per head does main pass, median and flags at once.
static bool small_call(const hqmq_encode_args* a) {
  const bool ext_med = a->median_mult > 0.f && a->med_in != nullptr;   // the median comes from the caller
  const int64_t tok = (int64_t)a->dst.B * a->T_new;
  return !ext_med && tok * a->dst.n_chunks <= kSmallMax && tok <= kSmallTok;
}

static int fill_small(const hqmq_encode_args* a, const WsPlan& wp, uint32_t* ws, SmallArgs& sa) {
  const hqmq_packed& d = a->dst;
  const bool med = a->median_mult > 0.f;
  const bool lut_ok = a->search == 0 && a->lut != nullptr && a->lut_footprint >= 0;
  if (lut_ok && ((uintptr_t)a->lut & 15)) return HQMQ_ERR_ALIGN;
  const unsigned char* lut_b = reinterpret_cast<const unsigned char*>(a->lut);
  sa.g = geom_of(a);
  sa.x = a->x; sa.qs = a->qs; sa.dst = d; sa.t_start = a->t_start; sa.joint = a->joint;
  sa.lut = lut_ok ? lut_b : nullptr;
  sa.nmul = lut_ok ? lut_b + kLutOffHeads + (size_t)d.H * kLutHeadBytes : nullptr;
  sa.C = a->median_mult; sa.med_out = a->med_out; sa.quantile = a->quantile;
  sa.status = ws + wp.status;
  sa.blk0 = wp.blk0; sa.nblk = wp.nblk;
  sa.scan = (med || d.ofrag) ? 1 : 0; sa.payload = med ? 1 : 0; sa.side = med ? 1 : 0;
  return HQMQ_OK;
}

extern "C" size_t hqmq_encode_pair_workspace_bytes(const hqmq_encode_args* k, const hqmq_encode_args* v) {
  const size_t wk = hqmq_encode_workspace_bytes(k), wv = hqmq_encode_workspace_bytes(v);
  if (!wk || !wv) return 0;
  return ((wk + 255) & ~(size_t)255) + wv;
}

extern "C" int hqmq_encode_pair(const hqmq_encode_args* k, const hqmq_encode_args* v, void* workspace, size_t workspace_bytes,
                                void* stream) {
  int rc = validate_encode(k);
  if (rc) return rc;
  rc = validate_encode(v);
  if (rc) return rc;
  const size_t wk = (plan_ws(*k).total + 255) & ~(size_t)255, wv = plan_ws(*v).total;
  if (!workspace || workspace_bytes < wk + wv) return HQMQ_ERR_WORKSPACE;
  if ((uintptr_t)workspace & 15) return HQMQ_ERR_ALIGN;
  unsigned char* wsb = reinterpret_cast<unsigned char*>(workspace);
  const hqmq_packed &dk = k->dst, &dv = v->dst;
  const bool same = dk.B == dv.B && dk.H == dv.H && dk.n_chunks == dv.n_chunks && k->T_new == v->T_new;
  if (!same || k->T_new == 0 || !small_call(k) || !small_call(v) || plan_ws(*k).nblk > kScanSmallBlocks ||
      plan_ws(*v).nblk > kScanSmallBlocks) {
    // no common launch shape: one tensor after the other, each with its part of the workspace
    rc = hqmq_encode(k, wsb, wk, stream);
    if (rc) return rc;
    return hqmq_encode(v, wsb + wk, wv, stream);
  }
  cudaStream_t st = (cudaStream_t)stream;
  SmallPair pr;
  rc = fill_small(k, plan_ws(*k), reinterpret_cast<uint32_t*>(wsb), pr.t[0]);
  if (rc) return rc;
  rc = fill_small(v, plan_ws(*v), reinterpret_cast<uint32_t*>(wsb + wk), pr.t[1]);
  if (rc) return rc;
  memcpy(pr.maps.ref_to_native, index_maps().ref_to_native, 24);
  // one launch for the whole append; the two status words (first word of each tensor's part) are cleared ahead of it
  HQMQ_CHECK_CUDA(cudaMemset2DAsync(wsb, wk, 0, sizeof(uint32_t), 2, st));
  append_pair_kernel<<<dim3(dk.H, 2), kSmallThreads, 0, st>>>(pr);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

extern "C" int hqmq_encode(const hqmq_encode_args* a, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = validate_encode(a);
  if (rc) return rc;
  if (a->T_new == 0) return HQMQ_OK;   // appending nothing: the planes stay as they are, no workspace needed
  const WsPlan wp = plan_ws(*a);
  if (!workspace || workspace_bytes < wp.total) return HQMQ_ERR_WORKSPACE;
  if ((uintptr_t)workspace & 15) return HQMQ_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  const hqmq_packed& d = a->dst;
  const bool med = a->median_mult > 0.f;
  const EncGeom g = geom_of(a);

  uint32_t* ws = reinterpret_cast<uint32_t*>(workspace);
  Maps24 maps;
  memcpy(maps.ref_to_native, index_maps().ref_to_native, 24);

  const bool ext_med = med && a->med_in != nullptr;   // the median comes from the caller (batch of a head split over GPUs)
  if (small_call(a)) {
    SmallArgs sa;
    rc = fill_small(a, wp, ws, sa);
    if (rc) return rc;
    encode_small_kernel<<<d.H, kSmallThreads, 0, st>>>(sa, maps);      // (clears the status word itself)
    if (sa.scan) scan_kernel<<<d.B * d.H, kScanWarps * 32, 0, st>>>(d, a->t_start, a->T_new, wp.blk0, wp.nblk, sa.payload, ws + wp.status);
    if (sa.side) side_kernel<<<dim3((wp.nblk + 7) / 8, d.B * d.H), 256, 0, st>>>(g, a->x, d, a->t_start, wp.blk0, wp.nblk);
    HQMQ_LAUNCH_CHECK();
    return HQMQ_OK;
  }
  HQMQ_CHECK_CUDA(cudaMemsetAsync(ws, 0, wp.zero_bytes, st));

  const int tok_per_block = kEncWarps * g.tpw * kEncIters;
  dim3 grid((a->T_new + tok_per_block - 1) / tok_per_block, d.B * d.H);
  const size_t smem_base = (size_t)g.S * 16 + (size_t)kEncWarps * g.tpw * kMaxRowWords * 4 + kHistBins * 4;
  if (smem_base > 200 * 1024) return HQMQ_ERR_UNSUPPORTED;
  // look-up-table search when a table is given and it fits shared memory next to the joint codebook
  // (lut_footprint: shared-memory bytes of the largest head's table, from hqmq_encode_lut_footprint; 0 = unknown:
  //  assume the largest a table can be)
  const size_t lut_foot = a->lut_footprint > 0 ? ((size_t)a->lut_footprint + 15) & ~(size_t)15
                                                : lut_smem_bytes(kLutNMax, kLutCellCap, kLutCandCap);
  const size_t smem_lut = smem_base + (size_t)24 * g.S * 16 + lut_foot;
  const bool use_lut = a->search == 0 && a->lut != nullptr && a->lut_footprint >= 0 && smem_lut <= 226 * 1024;
  // fast passes: d_head 128, 16-bit input, token rows on 16-byte boundaries (the fused last pass lists
  // undecided chunks by a 32-bit index over the (batch, token, chunk) grid of a head)
  // (d_head 64 with contiguous tokens runs the same kernels on pairs of tokens)
  const bool pair16 = pair16_of(*a);
  const int T32 = pair16 ? a->T_new / 2 : a->T_new;
  EncGeom g32 = g;
  if (pair16) { g32.n = 32; g32.npl = 32; g32.tpw = 1; g32.T_new = T32; g32.xs_t = 2 * g.xs_t; g32.pair16 = 1; }
  const bool fast32 = (g.n == 32 || pair16) && is_half_dtype(a->x_dtype) && ((uintptr_t)a->x & 15) == 0 && g.xs_b % 8 == 0 &&
                      g.xs_h % 8 == 0 && g.xs_t % 8 == 0 && (int64_t)d.B * a->T_new * 32 < ((int64_t)1 << 32);
  Fast32 f32{reinterpret_cast<const uint16_t*>(a->x), g.xs_b, g.xs_h, g32.xs_t, d.H, T32, pair16 ? 1 : 0};
  Fast32 f32_tok{reinterpret_cast<const uint16_t*>(a->x), g.xs_b, g.xs_h, g.xs_t, d.H, a->T_new, 0};   // per real token (the fix-up list)
  const Mul24& nmul = mul24_native();
  if (use_lut && (uintptr_t)a->lut & 15) return HQMQ_ERR_ALIGN;
  // specialised kernel: d_head 128, 16-bit input, one of the compiled field layouts
  const void* fastk = nullptr;
  const void* fastk_br = nullptr;
  bool predicted = false;
  const uint32_t* gate = nullptr;      // bracket mode: the word that sends the call through the multi-pass kernels after all
  if (use_lut && is_half_dtype(a->x_dtype) && (g.n == 32 || (pair16 && fast32))) {
    const bool h16 = a->x_dtype == HQMQ_F16;
#define HQMQ_PICK(IB_, RB_)                                                                              \
    if (g.ib == IB_ && g.rbits == RB_) {                                                                   \
      fastk = h16 ? (const void*)&encode_main32_kernel<HQMQ_F16, IB_, RB_, false>                          \
                  : (const void*)&encode_main32_kernel<HQMQ_BF16, IB_, RB_, false>;                        \
      fastk_br = h16 ? (const void*)&encode_main32_kernel<HQMQ_F16, IB_, RB_, true>                        \
                     : (const void*)&encode_main32_kernel<HQMQ_BF16, IB_, RB_, true>;                      \
    }
    HQMQ_PICK(10, 3) HQMQ_PICK(12, 4) HQMQ_PICK(13, 6)
#undef HQMQ_PICK
  }
  if (fastk) {
    const size_t smem_fast = (size_t)g.S * 16 + (size_t)kEnc32Warps * kMaxRowWords * 4 + 3 * kHistBins * 4 + (size_t)24 * g.S * 16 +
                             lut_foot + 16;
    const MainGrid mg = main_grid(T32, d.B, d.H);
    int iters = mg.iters;
    if (smem_fast > 48 * 1024) {
      HQMQ_CHECK_CUDA(cudaFuncSetAttribute(fastk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_fast));
      HQMQ_CHECK_CUDA(cudaFuncSetAttribute(fastk_br, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_fast));
    }
    dim3 fgrid(mg.gx, d.B * d.H);
    // Med3x: a sample of the tokens predicts the threshold statistic.  Two select levels over the sample give it
    // to 22 bits, the bracket pass then needs x only once; should the prediction fail, the multi-pass kernels
    // below (gated on a word the bracket's check raises) redo the call, with the sample's first level telling the
    // main pass which bins to refine.
    predicted = med && !ext_med && fast32 && T32 >= 1024;
    const bool bracket = predicted && bracket_wanted(*a) && wp.regions == (int)(fgrid.x * fgrid.y);
    const uint16_t* x16 = reinterpret_cast<const uint16_t*>(a->x);
    const unsigned char* lut_arg = reinterpret_cast<const unsigned char*>(a->lut);
    int t_start_arg = a->t_start;
    BracketArgs brargs{};
    if (predicted) {
      const int n_s = (T32 + kSampleStride - 1) / kSampleStride;
      const uint64_t N_s = (uint64_t)d.B * n_s * 32;
      int gs = (148 * 8 + d.B * d.H - 1) / (d.B * d.H);
      if (gs > (n_s + 15) / 16) gs = (n_s + 15) / 16;
      if (gs < 1) gs = 1;
      const bool h16s = a->x_dtype == HQMQ_F16;
      uint32_t* hist_s = ws + wp.hist_s;
      uint32_t* sel_s_w = ws + wp.sel_s;
      for (int level = 0; level < (bracket ? 2 : 1); ++level) {
        if (h16s) sample32_kernel<HQMQ_F16><<<dim3(gs, d.B * d.H), 256, 0, st>>>(f32, hist_s, level, sel_s_w);
        else sample32_kernel<HQMQ_BF16><<<dim3(gs, d.B * d.H), 256, 0, st>>>(f32, hist_s, level, sel_s_w);
        select_kernel<<<d.H, 256, 0, st>>>(hist_s, sel_s_w, level, N_s, a->median_mult, nullptr, nullptr, nullptr, nullptr,
                                           a->quantile, nullptr, 0);
      }
    }
    if (bracket) {
      const bool h16s = a->x_dtype == HQMQ_F16;
      uint32_t* sel_s_w = ws + wp.sel_s;
      const int n_s = (T32 + kSampleStride - 1) / kSampleStride;
      float delta = 3.0f / sqrtf((float)d.B * (float)n_s * 32.f);
      delta = delta < 0.002f ? 0.002f : delta > 0.012f ? 0.012f : delta;
      uint32_t* bp = ws + wp.bp;
      bracket_kernel<<<(d.H + 63) / 64, 64, 0, st>>>(sel_s_w, a->median_mult, delta, d.H, bp, ws + wp.band_b);
      gate = ws + wp.gate;
      brargs.bp = bp; brargs.bp_count = bp; brargs.band = ws + wp.band_b; brargs.und = ws + wp.und_b;
      brargs.rcnt = ws + wp.rcnt; brargs.rlist = ws + wp.rlist; brargs.histA = ws + wp.histA; brargs.rcap = wp.rcap; brargs.und_cap = wp.und_cap;
      brargs.run_if = nullptr;
      uint32_t* no_hist = nullptr;
      const uint32_t* no_sel = nullptr;
      void* kargs_b[] = {(void*)&g32, (void*)&x16, (void*)&a->qs, (void*)&d, (void*)&t_start_arg, (void*)&no_hist, (void*)&maps,
                         (void*)&a->joint, (void*)&lut_arg, (void*)&nmul, (void*)&iters, (void*)&no_sel, (void*)&brargs};
      HQMQ_CHECK_CUDA(cudaLaunchKernel(fastk_br, fgrid, dim3(kEnc32Threads), kargs_b, smem_fast, st));
      const uint64_t N_all = (uint64_t)d.B * a->T_new * d.n_chunks;
      list_pickA_kernel<<<d.H, 256, 0, st>>>(bp, ws + wp.histA, N_all, a->quantile, ws + wp.gate);
      list_histB_kernel<<<fgrid, 256, 0, st>>>(bp, ws + wp.rcnt, ws + wp.rlist, wp.rcap, d.H, ws + wp.histB, gate);
      list_pickB_kernel<<<d.H, 256, 0, st>>>(bp, ws + wp.histB, N_all, a->median_mult, a->quantile, ws + wp.sel_b, a->med_out, gate);
      int fg = (148 * 32 + d.B * d.H - 1) / (d.B * d.H);
      const int fg_max = (T32 + kF32Tok - 1) / kF32Tok;
      if (fg > fg_max) fg = fg_max;
      if (fg < 1) fg = 1;
      if (h16s) {
        fixup_list_kernel<HQMQ_F16><<<d.H, 256, 0, st>>>(f32_tok, d, a->t_start, g.ib, g.rbits, ws + wp.sel_b, ws + wp.band_b, ws + wp.und_b, gate, 0, wp.und_cap);
        fixup_scan_kernel<HQMQ_F16><<<dim3(fg, d.B * d.H), 256, 0, st>>>(f32, d, a->t_start, g.ib, g.rbits, ws + wp.sel_b, ws + wp.band_b, gate, 0, wp.und_cap);
      } else {
        fixup_list_kernel<HQMQ_BF16><<<d.H, 256, 0, st>>>(f32_tok, d, a->t_start, g.ib, g.rbits, ws + wp.sel_b, ws + wp.band_b, ws + wp.und_b, gate, 0, wp.und_cap);
        fixup_scan_kernel<HQMQ_BF16><<<dim3(fg, d.B * d.H), 256, 0, st>>>(f32, d, a->t_start, g.ib, g.rbits, ws + wp.sel_b, ws + wp.band_b, gate, 0, wp.und_cap);
      }
      brargs.run_if = gate;       // the multi-pass launch below runs only if the check raised the gate
    }
    const uint32_t* sel_s_arg = predicted ? ws + wp.sel_s : nullptr;
    uint32_t* hist_arg = med && !ext_med ? ws + wp.hist : nullptr;
    void* kargs[] = {(void*)&g32, (void*)&x16, (void*)&a->qs, (void*)&d, (void*)&t_start_arg, (void*)&hist_arg, (void*)&maps,
                     (void*)&a->joint, (void*)&lut_arg, (void*)&nmul, (void*)&iters, (void*)&sel_s_arg, (void*)&brargs};
    HQMQ_CHECK_CUDA(cudaLaunchKernel(fastk, fgrid, dim3(kEnc32Threads), kargs, smem_fast, st));
  } else if (use_lut) {
    if (smem_lut > 48 * 1024)
      HQMQ_CHECK_CUDA(cudaFuncSetAttribute(encode_main_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_lut));
    encode_main_kernel<true><<<grid, kEncThreads, smem_lut, st>>>(g, a->x, a->qs, d, a->t_start, med && !ext_med ? ws + wp.hist : nullptr,
                                                                  maps, a->joint, reinterpret_cast<const unsigned char*>(a->lut), nmul);
  } else {
    if (smem_base > 48 * 1024)
      HQMQ_CHECK_CUDA(cudaFuncSetAttribute(encode_main_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_base));
    encode_main_kernel<false><<<grid, kEncThreads, smem_base, st>>>(g, a->x, a->qs, d, a->t_start, med && !ext_med ? ws + wp.hist : nullptr,
                                                                    maps, a->joint, nullptr, nmul);
  }
  HQMQ_LAUNCH_CHECK();
  if (!med) {
    // no chunk of this call is flagged: the record offsets of its blocks just carry the running total on
    if (d.ofrag) {
      scan_kernel<<<d.B * d.H, kScanWarps * 32, 0, st>>>(d, a->t_start, a->T_new, wp.blk0, wp.nblk, 0, ws + wp.status);
      HQMQ_LAUNCH_CHECK();
    }
    return HQMQ_OK;
  }

  const uint64_t N = (uint64_t)d.B * a->T_new * d.n_chunks;
  const int64_t per_bh = (int64_t)a->T_new * d.n_chunks;
  // about 16 resident CTAs per SM in total; each CTA amortises zeroing and flushing its private histograms
  const int bh_count = d.B * d.H;
  int hb = (148 * 16 + bh_count - 1) / bh_count;
  const int hb_max = (int)((per_bh + 256 * 16 - 1) / (256 * 16));
  if (hb > hb_max) hb = hb_max;
  if (hb < 1) hb = 1;
  uint32_t* hist = ws + wp.hist;
  uint32_t* sel = ws + wp.sel;
  int fgrid = (148 * 32 + bh_count - 1) / bh_count;
  const int fgrid_max = (T32 + kF32Tok - 1) / kF32Tok;
  if (fgrid > fgrid_max) fgrid = fgrid_max;
  if (fgrid < 1) fgrid = 1;
  const dim3 f32_grid(fgrid, d.B * d.H);
  const bool h16 = a->x_dtype == HQMQ_F16;
  uint32_t* band = ws + wp.band;
  uint32_t* und = ws + wp.und;
  const uint32_t* sel_s = predicted ? ws + wp.sel_s : nullptr;
  uint32_t* hist_fb = ws + wp.hist_fb;
  if (ext_med) {
    // threshold from the caller's medians, then the plain flag pass (any geometry)
    thr_from_median_kernel<<<(d.H + 63) / 64, 64, 0, st>>>(a->med_in, a->median_mult, d.H, sel, a->med_out);
    const int tok_per_fblock = 8 * g.tpw;
    int fb = (a->T_new + 4 * tok_per_fblock - 1) / (4 * tok_per_fblock);
    const int fb_cap = (148 * 32 + bh_count - 1) / bh_count;
    if (fb > fb_cap) fb = fb_cap;
    if (fb < 1) fb = 1;
    flags_kernel<<<dim3(fb, d.B * d.H), 256, 0, st>>>(g, a->x, d, a->t_start, sel);
  } else {
  select_kernel<<<d.H, 256, 0, st>>>(hist, sel, 0, N, a->median_mult, nullptr, nullptr, nullptr, nullptr, a->quantile, gate, 1);
  if (fast32) {
    // (with a prediction this launch returns at once unless the sample named the wrong bins)
    if (h16) hist32_kernel<HQMQ_F16><<<f32_grid, 256, 0, st>>>(f32, hist, sel, 1, sel_s, hist_fb, gate, 1);
    else hist32_kernel<HQMQ_BF16><<<f32_grid, 256, 0, st>>>(f32, hist, sel, 1, sel_s, hist_fb, gate, 1);
    select_kernel<<<d.H, 256, 0, st>>>(hist, sel, 1, N, a->median_mult, nullptr, band, sel_s, hist_fb, a->quantile, gate, 1);
    // last histogram level and provisional flags in one pass, exact threshold, then the (normally empty) fix-up
    if (h16) histflags32_kernel<HQMQ_F16><<<f32_grid, 256, 0, st>>>(f32, d, a->t_start, g.ib, g.rbits, hist, sel, band, und, gate, 1);
    else histflags32_kernel<HQMQ_BF16><<<f32_grid, 256, 0, st>>>(f32, d, a->t_start, g.ib, g.rbits, hist, sel, band, und, gate, 1);
    select_kernel<<<d.H, 256, 0, st>>>(hist, sel, 2, N, a->median_mult, a->med_out, nullptr, nullptr, nullptr, a->quantile, gate, 1);
    if (h16) {
      fixup_list_kernel<HQMQ_F16><<<d.H, 256, 0, st>>>(f32_tok, d, a->t_start, g.ib, g.rbits, sel, band, und, gate, 1, kUndCap);
      fixup_scan_kernel<HQMQ_F16><<<f32_grid, 256, 0, st>>>(f32, d, a->t_start, g.ib, g.rbits, sel, band, gate, 1, kUndCap);
    } else {
      fixup_list_kernel<HQMQ_BF16><<<d.H, 256, 0, st>>>(f32_tok, d, a->t_start, g.ib, g.rbits, sel, band, und, gate, 1, kUndCap);
      fixup_scan_kernel<HQMQ_BF16><<<f32_grid, 256, 0, st>>>(f32, d, a->t_start, g.ib, g.rbits, sel, band, gate, 1, kUndCap);
    }
  } else {
    hist_kernel<<<dim3(hb, d.B * d.H), 256, 0, st>>>(g, a->x, hist, sel, 1);
    select_kernel<<<d.H, 256, 0, st>>>(hist, sel, 1, N, a->median_mult, nullptr, nullptr, nullptr, nullptr, a->quantile, nullptr, 0);
    hist_kernel<<<dim3(hb, d.B * d.H), 256, 0, st>>>(g, a->x, hist, sel, 2);
    select_kernel<<<d.H, 256, 0, st>>>(hist, sel, 2, N, a->median_mult, a->med_out, nullptr, nullptr, nullptr, a->quantile, nullptr, 0);
    const int tok_per_fblock = 8 * g.tpw;
    int fb = (a->T_new + 4 * tok_per_fblock - 1) / (4 * tok_per_fblock);
    const int fb_cap = (148 * 32 + bh_count - 1) / bh_count;
    if (fb > fb_cap) fb = fb_cap;
    if (fb < 1) fb = 1;
    flags_kernel<<<dim3(fb, d.B * d.H), 256, 0, st>>>(g, a->x, d, a->t_start, sel);
  }
  }
  HQMQ_LAUNCH_CHECK();
  scan_kernel<<<d.B * d.H, kScanWarps * 32, 0, st>>>(d, a->t_start, a->T_new, wp.blk0, wp.nblk, 1, ws + wp.status);
  side_kernel<<<dim3((wp.nblk + 7) / 8, d.B * d.H), 256, 0, st>>>(g, a->x, d, a->t_start, wp.blk0, wp.nblk);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}
