// Shared host/device helpers for the hqmq_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hqmq_b200.h"

#define HQMQ_CHECK_CUDA(expr)                    \
  do {                                           \
    cudaError_t e__ = (expr);                    \
    if (e__ != cudaSuccess) return HQMQ_ERR_CUDA; \
  } while (0)

#define HQMQ_LAUNCH_CHECK()                                  \
  do {                                                       \
    if (cudaGetLastError() != cudaSuccess) return HQMQ_ERR_CUDA; \
  } while (0)

namespace hqmq {

// ---- the 24 Hurwitz units and the factorisation p = u * omega^a -----------------------
// Reference order of the primary codebook: index 2*axis + (sign<0) for the 8 axis units,
// 8 + sum_i (sign_i<0) << (3-i) for the 16 half-integer units.
struct IndexMaps {
  uint8_t ref_to_native[24];  // p -> (a << 3) | u
  uint8_t native_to_ref[24];  // (a << 3) | u -> p
};
const IndexMaps& index_maps();

__host__ __device__ inline int idx_bits_for(int S) {
  int k = 24 * S, b = 0;
  while ((1 << b) < k) ++b;
  return b;
}
__host__ __device__ inline int row_bytes_for(int n_chunks, int S, int radius_bits) {
  int bits = n_chunks * (idx_bits_for(S) + radius_bits);
  return ((bits + 31) / 32) * 4;
}

// native_idx = ((a*S + s) << 3) | u   <->   reference k = p*S + s
__host__ __device__ inline int native_from_ref(int k, int S, const uint8_t* ref_to_native) {
  int p = k / S, s = k - p * S;
  int au = ref_to_native[p];
  return (((au >> 3) * S + s) << 3) | (au & 7);
}
__host__ __device__ inline int ref_from_native(int ni, int S, const uint8_t* native_to_ref) {
  int u = ni & 7, m = ni >> 3;
  int a = m / S, s = m - a * S;
  return native_to_ref[(a << 3) | u] * S + s;
}

// ---- element access --------------------------------------------------------------------
__device__ __forceinline__ float bits16_to_float(uint16_t v, int dtype) {
  if (dtype == HQMQ_F16) return __half2float(__ushort_as_half(v));
  return __bfloat162float(__ushort_as_bfloat16(v));
}
__device__ __forceinline__ uint16_t float_to_bits16(float f, int dtype) {
  if (dtype == HQMQ_F16) return __half_as_ushort(__float2half_rn(f));
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ float load_float(const void* p, int64_t i, int dtype) {
  if (dtype == HQMQ_F32) return reinterpret_cast<const float*>(p)[i];
  return bits16_to_float(reinterpret_cast<const uint16_t*>(p)[i], dtype);
}
__device__ __forceinline__ void store_float(void* p, int64_t i, float v, int dtype) {
  if (dtype == HQMQ_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<uint16_t*>(p)[i] = float_to_bits16(v, dtype);
}
__device__ __forceinline__ long long load_int(const void* p, int64_t i, int dtype) {
  switch (dtype) {
    case HQMQ_I32: return reinterpret_cast<const int32_t*>(p)[i];
    case HQMQ_I16: return reinterpret_cast<const int16_t*>(p)[i];
    case HQMQ_I8: return reinterpret_cast<const int8_t*>(p)[i];
    case HQMQ_U8: return reinterpret_cast<const uint8_t*>(p)[i];
    default: return reinterpret_cast<const long long*>(p)[i];
  }
}
inline int dtype_size(int dtype) {
  switch (dtype) {
    case HQMQ_F32: case HQMQ_I32: return 4;
    case HQMQ_F16: case HQMQ_BF16: case HQMQ_I16: return 2;
    case HQMQ_I8: case HQMQ_U8: return 1;
    case HQMQ_I64: return 8;
    default: return 0;
  }
}
inline bool is_float_dtype(int dt) { return dt == HQMQ_F32 || dt == HQMQ_F16 || dt == HQMQ_BF16; }
inline bool is_half_dtype(int dt) { return dt == HQMQ_F16 || dt == HQMQ_BF16; }

// ---- bit fields of a packed code row ------------------------------------------------------
// Field c of width cb at bit c*cb of a little-endian row of 32-bit words.
__device__ __forceinline__ uint32_t row_field(const uint32_t* row, int c, int cb) {
  int bit = c * cb;
  int w = bit >> 5, sh = bit & 31;
  uint32_t lo = row[w];
  uint32_t hi = (sh + cb > 32) ? row[w + 1] : 0u;
  return __funnelshift_r(lo, hi, sh) & ((1u << cb) - 1u);
}

// Per-token radius scale of a native tensor (fp16 / bf16 / fp32 plane).
__device__ __forceinline__ float load_scale(const hqmq_packed& p, int64_t row) {
  if (p.scale_dtype == HQMQ_F32) return reinterpret_cast<const float*>(p.rs)[row];
  return bits16_to_float(reinterpret_cast<const uint16_t*>(p.rs)[row], p.scale_dtype);
}
__device__ __forceinline__ void store_scale(const hqmq_packed& p, int64_t row, float v) {
  if (p.scale_dtype == HQMQ_F32) reinterpret_cast<float*>(p.rs)[row] = v;
  else reinterpret_cast<uint16_t*>(p.rs)[row] = float_to_bits16(v, p.scale_dtype);
}

// Validation of a native descriptor (host).
int check_packed(const hqmq_packed& p, bool need_flags);

__host__ __device__ inline int64_t packed_rows(const hqmq_packed& p) { return (int64_t)p.B * p.H * p.T_cap; }

}  // namespace hqmq
