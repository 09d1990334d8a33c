// Decode-attention kernels for the native layouts with a compile-time field layout:
// (index bits, radius bits) = (10,3) s24_r3, (12,4) s96_r4, (13,6) s192_r6; d_head 64 or 128; G <= 8.
#include "attn_tma.cuh"

namespace hqmq {
namespace attn {

// One CTA per SM; its warps share the codeword tables and each streams its own tiles through
// shared memory with bulk asynchronous copies.
template <int N, int IB, int RB, bool OUTL>
__global__ void __launch_bounds__(OUTL ? kFastWarpsOutl * 32 : kFastWarps * 32, 1) attn_fast_kernel(const AttnParams p) {
  attn_decode_tma_body<N, IB, RB, OUTL ? kFastWarpsOutl : kFastWarps, OUTL>(p, p.status);
}

// Shared memory of one warp's staging ring (must match StageLayout).
size_t fast_warp_bytes(int n_chunks, int ib, int rb, bool outl) {
  const size_t row = (size_t)n_chunks * (ib + rb) / 8;
  const size_t stage = 2 * kTile * row + 64 + (outl ? 128 + kSideK + (kPay + 2) * 8 + 16 : 0);
  const size_t merge = (size_t)8 * (4 * n_chunks + 2) * 4;   // one warp's partial during the in-CTA merge
  return kStages * stage > merge ? kStages * stage : merge;
}

template <int N, int IB, int RB, bool OUTL>
static const void* fn() { return reinterpret_cast<const void*>(&attn_fast_kernel<N, IB, RB, OUTL>); }

template <int N, bool OUTL>
static const void* pick(int ib, int rb) {
  if (ib == 10 && rb == 3) return fn<N, 10, 3, OUTL>();
  if (ib == 12 && rb == 4) return fn<N, 12, 4, OUTL>();
  if (ib == 13 && rb == 6) return fn<N, 13, 6, OUTL>();
  return nullptr;
}

// Kernel for (n_chunks, idx bits, radius bits, outliers) or nullptr when no specialisation exists.
const void* fast_kernel(int n_chunks, int ib, int rb, bool outl) {
  if ((n_chunks * (ib + rb)) % 32) return nullptr;   // rows must be whole words without padding
  if (n_chunks == 32) return outl ? pick<32, true>(ib, rb) : pick<32, false>(ib, rb);
  if (n_chunks == 16) return outl ? pick<16, true>(ib, rb) : pick<16, false>(ib, rb);
  return nullptr;
}

}  // namespace attn
}  // namespace hqmq
