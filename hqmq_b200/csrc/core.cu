// Library entry points that are not on the two hot kernels: error strings, device check,
// index maps, codebook tables, layout conversion (pack / unpack) and packed dequant.
#include <math.h>
#include <string.h>

#include "common.cuh"

namespace hqmq {

// ---------------------------------------------------------------------------------------
// p = u * omega^a factorisation of the 24 Hurwitz units
// ---------------------------------------------------------------------------------------
namespace {
struct Quat { double w, x, y, z; };
Quat qmul(const Quat& a, const Quat& b) {
  return {a.w * b.w - a.x * b.x - a.y * b.y - a.z * b.z, a.w * b.x + a.x * b.w + a.y * b.z - a.z * b.y,
          a.w * b.y - a.x * b.z + a.y * b.w + a.z * b.x, a.w * b.z + a.x * b.y - a.y * b.x + a.z * b.w};
}
Quat primary(int p) {
  double v[4] = {0, 0, 0, 0};
  if (p < 8) {
    v[p >> 1] = (p & 1) ? -1.0 : 1.0;
  } else {
    int bits = p - 8;
    for (int i = 0; i < 4; ++i) v[i] = ((bits >> (3 - i)) & 1) ? -0.5 : 0.5;
  }
  return {v[0], v[1], v[2], v[3]};
}
IndexMaps build_maps() {
  IndexMaps m;
  memset(&m, 0xff, sizeof(m));
  Quat omega = primary(8);
  Quat pw[3] = {primary(0), omega, qmul(omega, omega)};
  for (int a = 0; a < 3; ++a)
    for (int u = 0; u < 8; ++u) {
      Quat q = qmul(primary(u), pw[a]);
      for (int p = 0; p < 24; ++p) {
        Quat r = primary(p);
        if (fabs(r.w - q.w) + fabs(r.x - q.x) + fabs(r.y - q.y) + fabs(r.z - q.z) < 1e-9) {
          m.ref_to_native[p] = (uint8_t)((a << 3) | u);
          m.native_to_ref[(a << 3) | u] = (uint8_t)p;
        }
      }
    }
  return m;
}
}  // namespace

const IndexMaps& index_maps() {
  static const IndexMaps m = build_maps();
  return m;
}

int check_packed(const hqmq_packed& p, bool need_flags) {
  if (p.struct_size != sizeof(hqmq_packed)) return HQMQ_ERR_ARG;
  if (p.B <= 0 || p.H <= 0 || p.T_cap <= 0 || (p.T_cap % HQMQ_T_ALIGN)) return HQMQ_ERR_SHAPE;
  if (p.n_chunks < 1 || p.n_chunks > 32) return HQMQ_ERR_SHAPE;
  if (p.S < 1 || 24 * p.S > 65536 || p.radius_bits < 1 || p.radius_bits > 8) return HQMQ_ERR_SHAPE;
  if (p.row_bytes != row_bytes_for(p.n_chunks, p.S, p.radius_bits)) return HQMQ_ERR_SHAPE;
  if (!is_float_dtype(p.scale_dtype)) return HQMQ_ERR_DTYPE;
  if (!p.codes || !p.rs) return HQMQ_ERR_ARG;
  if (((uintptr_t)p.codes & 15) || ((uintptr_t)p.rs & 15)) return HQMQ_ERR_ALIGN;
  if (need_flags || p.flags) {
    if (!p.flags || !p.out_vals || !p.out_off || !p.out_count) return HQMQ_ERR_ARG;
    if (!is_float_dtype(p.out_dtype) || p.out_cap < 0) return HQMQ_ERR_DTYPE;
    // payload entries are read as one 8-byte (16-bit values) or 16-byte (fp32 values) load
    if (((uintptr_t)p.flags & 15) || ((uintptr_t)p.out_vals & (p.out_dtype == HQMQ_F32 ? 15 : 7))) return HQMQ_ERR_ALIGN;
  }
  if (p.ofrag) {
    if (!p.flags || !p.ofrag_off || p.ofrag_cap < 0) return HQMQ_ERR_ARG;
    if (((uintptr_t)p.ofrag & 15) || ((uintptr_t)p.ofrag_off & 3)) return HQMQ_ERR_ALIGN;
  }
  return HQMQ_OK;
}

struct Maps24 { uint8_t ref_to_native[24]; uint8_t native_to_ref[24]; };
static Maps24 maps_arg() {
  Maps24 m;
  memcpy(m.ref_to_native, index_maps().ref_to_native, 24);
  memcpy(m.native_to_ref, index_maps().native_to_ref, 24);
  return m;
}

// ---------------------------------------------------------------------------------------
// codebook tables
// ---------------------------------------------------------------------------------------
__global__ void codebook_tables_kernel(const float* __restrict__ joint, int H, int S, uint16_t* __restrict__ table16,
                                       Maps24 maps) {
  int K = 24 * S;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)H * K) return;
  int h = (int)(i / K), ni = (int)(i - (int64_t)h * K);
  int k = ref_from_native(ni, S, maps.native_to_ref);
  const float4 c = reinterpret_cast<const float4*>(joint)[(int64_t)h * K + k];
  ushort4 o;
  o.x = __half_as_ushort(__float2half_rn(c.x));
  o.y = __half_as_ushort(__float2half_rn(c.y));
  o.z = __half_as_ushort(__float2half_rn(c.z));
  o.w = __half_as_ushort(__float2half_rn(c.w));
  reinterpret_cast<ushort4*>(table16)[i] = o;
}

// ---------------------------------------------------------------------------------------
// unpack: native -> reference tuple
// ---------------------------------------------------------------------------------------
__global__ void unpack_kernel(hqmq_packed p, int t0, int T, int32_t* __restrict__ idx, int32_t* __restrict__ rq,
                              float* __restrict__ rs, uint8_t* __restrict__ flags, Maps24 maps) {
  const int n = p.n_chunks;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)p.B * p.H * T * n;
  if (i >= total) return;
  int c = (int)(i % n);
  int64_t tok = i / n;  // (b*H + h)*T + t
  int t = (int)(tok % T);
  int64_t bh = tok / T;
  int64_t row = bh * p.T_cap + t0 + t;
  const int ib = idx_bits_for(p.S), cb = ib + p.radius_bits;
  const uint32_t* rowp = reinterpret_cast<const uint32_t*>(p.codes + row * p.row_bytes);
  uint32_t f = row_field(rowp, c, cb);
  idx[i] = ref_from_native((int)(f & ((1u << ib) - 1u)), p.S, maps.native_to_ref);
  rq[i] = (int32_t)(f >> ib);
  if (c == 0) rs[tok] = load_scale(p, row);
  if (flags) flags[i] = p.flags ? (uint8_t)((p.flags[row] >> c) & 1u) : 0;
}

// ---------------------------------------------------------------------------------------
// pack: reference tuple -> native rows (one thread per token)
// ---------------------------------------------------------------------------------------
__global__ void pack_kernel(hqmq_ref_packed s, int T, hqmq_packed p, int t_start, Maps24 maps) {
  int64_t tok = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (tok >= (int64_t)p.B * p.H * T) return;
  int t = (int)(tok % T);
  int64_t bh = tok / T;
  int h = (int)(bh % p.H), b = (int)(bh / p.H);
  const int n = p.n_chunks, ib = idx_bits_for(p.S), cb = ib + p.radius_bits;
  uint32_t words[25];   // up to 32 chunks x (16 index + 8 radius) bits = 24 words
  const int nw = p.row_bytes / 4;
  for (int w = 0; w < nw; ++w) words[w] = 0;
  int64_t ib0 = b * s.idx_stride[0] + h * s.idx_stride[1] + t * s.idx_stride[2];
  int64_t rb0 = b * s.rq_stride[0] + h * s.rq_stride[1] + t * s.rq_stride[2];
  for (int c = 0; c < n; ++c) {
    int k = (int)load_int(s.idx, ib0 + c, s.idx_dtype);
    k = k < 0 ? 0 : (k >= 24 * p.S ? 24 * p.S - 1 : k);
    uint32_t r = (uint32_t)load_int(s.rq, rb0 + c, s.rq_dtype) & ((1u << p.radius_bits) - 1u);
    uint32_t f = (uint32_t)native_from_ref(k, p.S, maps.ref_to_native) | (r << ib);
    int bit = c * cb, w = bit >> 5, sh = bit & 31;
    words[w] |= f << sh;
    if (sh + cb > 32) words[w + 1] |= f >> (32 - sh);
  }
  int64_t row = bh * p.T_cap + t_start + t;
  uint32_t* rowp = reinterpret_cast<uint32_t*>(p.codes + row * p.row_bytes);
  for (int w = 0; w < nw; ++w) rowp[w] = words[w];
  float rs = load_float(s.rs, b * s.rs_stride[0] + h * s.rs_stride[1] + t, s.rs_dtype);
  store_scale(p, row, rs);
  if (p.flags) p.flags[row] = 0u;
}

// ---------------------------------------------------------------------------------------
// dequant
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float round_to(float v, int dtype) {
  if (dtype == HQMQ_F16) return __half2float(__float2half_rn(v));
  if (dtype == HQMQ_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}

// Position of flagged chunk (row, c) in the outlier payload of its (b,h).
__device__ __forceinline__ uint32_t outlier_slot(const hqmq_packed& p, int64_t bh, int t, int c) {
  const int blk = t / HQMQ_OUT_BLOCK;
  const int nblk = p.T_cap / HQMQ_OUT_BLOCK + 1;
  uint32_t off = p.out_off[bh * nblk + blk];
  const uint32_t* fl = p.flags + bh * p.T_cap;
  for (int tt = blk * HQMQ_OUT_BLOCK; tt < t; ++tt) off += __popc(fl[tt]);
  off += __popc(fl[t] & ((1u << c) - 1u));
  return off;
}

__global__ void dequant_native_kernel(hqmq_packed p, int t0, int T, const float* __restrict__ joint, int r_qmax,
                                      int scale_first, int out_dtype, void* __restrict__ out, int merge, Maps24 maps) {
  const int n = p.n_chunks;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)p.B * p.H * T * n) return;
  int c = (int)(i % n);
  int64_t tok = i / n;
  int t = (int)(tok % T);
  int64_t bh = tok / T;
  int h = (int)(bh % p.H);
  int64_t row = bh * p.T_cap + t0 + t;
  const int ib = idx_bits_for(p.S), cb = ib + p.radius_bits;
  float v[4];
  if (merge && p.flags && ((p.flags[row] >> c) & 1u)) {
    // an entry beyond the side buffer's capacity was dropped by the encoder: it reads as 0
    uint32_t slot = outlier_slot(p, bh, t0 + t, c);
    const int64_t o = ((int64_t)bh * p.out_cap + slot) * 4;
    for (int e = 0; e < 4; ++e) v[e] = slot < (uint32_t)p.out_cap ? load_float(p.out_vals, o + e, p.out_dtype) : 0.f;
  } else {
    const uint32_t* rowp = reinterpret_cast<const uint32_t*>(p.codes + row * p.row_bytes);
    uint32_t f = row_field(rowp, c, cb);
    int k = ref_from_native((int)(f & ((1u << ib) - 1u)), p.S, maps.native_to_ref);
    float rq = (float)(f >> ib);
    float rs = load_scale(p, row);
    float radius = scale_first ? __fmul_rn(rq, __fdiv_rn(rs, (float)r_qmax)) : __fdiv_rn(__fmul_rn(rq, rs), (float)r_qmax);
    const float4 cw = reinterpret_cast<const float4*>(joint)[(int64_t)h * 24 * p.S + k];
    v[0] = __fmul_rn(cw.x, radius); v[1] = __fmul_rn(cw.y, radius);
    v[2] = __fmul_rn(cw.z, radius); v[3] = __fmul_rn(cw.w, radius);
  }
  for (int e = 0; e < 4; ++e) store_float(out, i * 4 + e, v[e], out_dtype);
}

__global__ void dequant_ref_kernel(hqmq_ref_packed s, int B, int H, int T, int n, const void* __restrict__ joint,
                                   int joint_dtype, int K, int r_qmax, int scale_first, int compute_dtype,
                                   int out_dtype, void* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)B * H * T * n) return;
  int c = (int)(i % n);
  int64_t tok = i / n;
  int t = (int)(tok % T);
  int64_t bh = tok / T;
  int h = (int)(bh % H), b = (int)(bh / H);
  long long k = load_int(s.idx, b * s.idx_stride[0] + h * s.idx_stride[1] + t * s.idx_stride[2] + c, s.idx_dtype);
  if (k < 0) k = 0;
  if (k >= K) k = K - 1;
  float rq = (float)load_int(s.rq, b * s.rq_stride[0] + h * s.rq_stride[1] + t * s.rq_stride[2] + c, s.rq_dtype);
  float rs = load_float(s.rs, b * s.rs_stride[0] + h * s.rs_stride[1] + t, s.rs_dtype);
  float radius;
  if (scale_first) radius = round_to(__fmul_rn(rq, round_to(__fdiv_rn(rs, (float)r_qmax), compute_dtype)), compute_dtype);
  else radius = round_to(__fdiv_rn(round_to(__fmul_rn(rq, rs), compute_dtype), (float)r_qmax), compute_dtype);
  for (int e = 0; e < 4; ++e) {
    float cw = load_float(joint, ((int64_t)h * K + k) * 4 + e, joint_dtype);
    store_float(out, i * 4 + e, round_to(__fmul_rn(cw, radius), compute_dtype), out_dtype);
  }
}

}  // namespace hqmq

using namespace hqmq;

extern "C" {

int hqmq_abi_version(void) { return HQMQ_ABI_VERSION; }

int hqmq_read_status(const void* workspace, uint32_t* status, void* stream) {
  if (!workspace || !status) return HQMQ_ERR_ARG;
  HQMQ_CHECK_CUDA(cudaMemcpyAsync(status, workspace, sizeof(uint32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  HQMQ_CHECK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return HQMQ_OK;
}

const char* hqmq_strerror(int code) {
  switch (code) {
    case HQMQ_OK: return "ok";
    case HQMQ_ERR_ARG: return "invalid argument (null pointer, struct_size or enum)";
    case HQMQ_ERR_SHAPE: return "unsupported or inconsistent shape";
    case HQMQ_ERR_DTYPE: return "unsupported element type";
    case HQMQ_ERR_ALIGN: return "pointer or stride not aligned as required";
    case HQMQ_ERR_WORKSPACE: return "workspace missing or too small";
    case HQMQ_ERR_ARCH: return "device is not compute capability 10.x (sm_100a required)";
    case HQMQ_ERR_CUDA: return "CUDA runtime error";
    case HQMQ_ERR_UNSUPPORTED: return "configuration not supported";
    case HQMQ_ERR_CAPACITY: return "packed cache or outlier buffer capacity exceeded";
    case HQMQ_ERR_STATIC_SCRATCH:
      return "the problem needs more scratch than the library's built-in buffer; call hqmq_attn_decode with a workspace";
    case HQMQ_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    default: return "unknown error";
  }
}

int hqmq_device_check(int device) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) return HQMQ_ERR_CUDA;
  return major == 10 ? HQMQ_OK : HQMQ_ERR_ARCH;
}

int hqmq_idx_bits(int S) { return (S < 1 || 24 * S > 65536) ? HQMQ_ERR_SHAPE : idx_bits_for(S); }

int hqmq_row_bytes(int n_chunks, int S, int radius_bits) {
  if (n_chunks < 1 || n_chunks > 32 || S < 1 || 24 * S > 65536 || radius_bits < 1 || radius_bits > 8) return HQMQ_ERR_SHAPE;
  return row_bytes_for(n_chunks, S, radius_bits);
}

int hqmq_native_index_maps(uint8_t* ref_to_native, uint8_t* native_to_ref) {
  if (!ref_to_native || !native_to_ref) return HQMQ_ERR_ARG;
  memcpy(ref_to_native, index_maps().ref_to_native, 24);
  memcpy(native_to_ref, index_maps().native_to_ref, 24);
  return HQMQ_OK;
}

int hqmq_codebook_tables(const float* joint, int H, int S, uint16_t* table16, void* stream) {
  if (!joint || !table16) return HQMQ_ERR_ARG;
  if (H < 1 || S < 1 || 24 * S > 65536) return HQMQ_ERR_SHAPE;
  if (((uintptr_t)joint & 15) || ((uintptr_t)table16 & 7)) return HQMQ_ERR_ALIGN;
  int64_t n = (int64_t)H * 24 * S;
  codebook_tables_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(joint, H, S, table16, maps_arg());
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

int hqmq_unpack(const hqmq_packed* src, int t0, int T, int32_t* idx, int32_t* rq, float* rs, uint8_t* flags,
                void* stream) {
  if (!src || !idx || !rq || !rs) return HQMQ_ERR_ARG;
  int rc = check_packed(*src, false);
  if (rc) return rc;
  if (t0 < 0 || T < 0 || t0 + T > src->T_cap) return HQMQ_ERR_SHAPE;
  int64_t n = (int64_t)src->B * src->H * T * src->n_chunks;
  if (n == 0) return HQMQ_OK;
  unpack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(*src, t0, T, idx, rq, rs, flags, maps_arg());
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

static int check_ref(const hqmq_ref_packed& s) {
  if (s.struct_size != sizeof(hqmq_ref_packed)) return HQMQ_ERR_ARG;
  if (!s.idx || !s.rq || !s.rs) return HQMQ_ERR_ARG;
  if (!(s.idx_dtype == HQMQ_I32 || s.idx_dtype == HQMQ_I64 || s.idx_dtype == HQMQ_I16)) return HQMQ_ERR_DTYPE;
  if (!(s.rq_dtype == HQMQ_I32 || s.rq_dtype == HQMQ_I16 || s.rq_dtype == HQMQ_I8 || s.rq_dtype == HQMQ_U8 ||
        s.rq_dtype == HQMQ_I64))
    return HQMQ_ERR_DTYPE;
  if (!is_float_dtype(s.rs_dtype)) return HQMQ_ERR_DTYPE;
  return HQMQ_OK;
}

int hqmq_pack(const hqmq_ref_packed* src, int T, hqmq_packed* dst, int t_start, void* stream) {
  if (!src || !dst) return HQMQ_ERR_ARG;
  int rc = check_ref(*src);
  if (rc) return rc;
  rc = check_packed(*dst, false);
  if (rc) return rc;
  if (t_start < 0 || T < 0 || t_start + T > dst->T_cap) return HQMQ_ERR_CAPACITY;
  int64_t n = (int64_t)dst->B * dst->H * T;
  if (n == 0) return HQMQ_OK;
  pack_kernel<<<(unsigned)((n + 127) / 128), 128, 0, (cudaStream_t)stream>>>(*src, T, *dst, t_start, maps_arg());
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

int hqmq_dequant(const hqmq_dequant_args* a, void* stream) {
  if (!a || a->struct_size != sizeof(hqmq_dequant_args) || !a->out) return HQMQ_ERR_ARG;
  if (!is_float_dtype(a->out_dtype)) return HQMQ_ERR_DTYPE;
  if (a->r_qmax < 1) return HQMQ_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (a->layout == 0) {
    int rc = check_packed(a->src_native, a->merge_outliers != 0 && a->src_native.flags != nullptr);
    if (rc) return rc;
    if (!a->joint_f32) return HQMQ_ERR_ARG;
    if ((uintptr_t)a->joint_f32 & 15) return HQMQ_ERR_ALIGN;
    if (a->t0 < 0 || a->T < 0 || a->t0 + a->T > a->src_native.T_cap) return HQMQ_ERR_SHAPE;
    int64_t n = (int64_t)a->src_native.B * a->src_native.H * a->T * a->src_native.n_chunks;
    if (n == 0) return HQMQ_OK;
    dequant_native_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a->src_native, a->t0, a->T, a->joint_f32, a->r_qmax,
                                                                    a->scale_first, a->out_dtype, a->out,
                                                                    a->merge_outliers, maps_arg());
  } else if (a->layout == 1) {
    int rc = check_ref(a->src_ref);
    if (rc) return rc;
    if (!a->joint || !is_float_dtype(a->joint_dtype)) return HQMQ_ERR_ARG;
    if (a->B < 0 || a->H < 1 || a->T < 0 || a->n_chunks < 1 || a->K < 1) return HQMQ_ERR_SHAPE;
    int64_t n = (int64_t)a->B * a->H * a->T * a->n_chunks;
    if (n == 0) return HQMQ_OK;
    // arithmetic is done in the promoted type of joint and rs, as torch would
    int cd = (a->joint_dtype == a->src_ref.rs_dtype) ? a->joint_dtype : HQMQ_F32;
    dequant_ref_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a->src_ref, a->B, a->H, a->T, a->n_chunks, a->joint,
                                                                 a->joint_dtype, a->K, a->r_qmax, a->scale_first, cd,
                                                                 a->out_dtype, a->out);
  } else {
    return HQMQ_ERR_ARG;
  }
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

}  // extern "C"
