// Decode-attention kernels with one CTA-wide staging ring (long key ranges), native layouts with a compile-time
// field layout: (index bits, radius bits) = (10,3) s24_r3, (12,4) s96_r4, (13,6) s192_r6; d_head 64 or 128; G <= 8.
#include "attn_ring.cuh"

namespace hqmq {
namespace attn {

// SDT: element type of the per-token scale planes (HQMQ_F16 or HQMQ_BF16), fixed at compile time like the field layout.
template <int N, int IB, int RB, bool OUTL, int SDT>
__global__ void __launch_bounds__((ring_warps(N) + 1) * 32, 1) attn_ring_kernel(const AttnParams p) {
  attn_ring_body<N, IB, RB, OUTL, SDT>(p);
}

template <int N, int IB, int RB, bool OUTL>
static void fill(int sdt, RingKernelInfo& k) {
  k.fn = sdt == HQMQ_F16 ? reinterpret_cast<const void*>(&attn_ring_kernel<N, IB, RB, OUTL, HQMQ_F16>)
                         : reinterpret_cast<const void*>(&attn_ring_kernel<N, IB, RB, OUTL, HQMQ_BF16>);
  k.stage_bytes = RingLayout<N, IB, RB, OUTL>::BYTES;
  k.warps = ring_warps(N);
}

template <int N, bool OUTL>
static bool pick(int ib, int rb, int sdt, RingKernelInfo& k) {
  if (ib == 10 && rb == 3) { fill<N, 10, 3, OUTL>(sdt, k); return true; }
  if (ib == 12 && rb == 4) { fill<N, 12, 4, OUTL>(sdt, k); return true; }
  if (ib == 13 && rb == 6) { fill<N, 13, 6, OUTL>(sdt, k); return true; }
  return false;
}

// Kernel for (n_chunks, idx bits, radius bits, outliers, scale dtype); false when no specialisation exists.
bool ring_kernel(int n_chunks, int ib, int rb, bool outl, int scale_dtype, RingKernelInfo& k) {
  if ((n_chunks * (ib + rb)) % 32) return false;   // rows must be whole words without padding
  if (scale_dtype != HQMQ_F16 && scale_dtype != HQMQ_BF16) return false;
  if (n_chunks == 32) return outl ? pick<32, true>(ib, rb, scale_dtype, k) : pick<32, false>(ib, rb, scale_dtype, k);
  if (n_chunks == 16) return outl ? pick<16, true>(ib, rb, scale_dtype, k) : pick<16, false>(ib, rb, scale_dtype, k);
  return false;
}

size_t ring_smem_total(int table_rows, int repk_log2, int repv_log2, int d, bool outl, int stages, int merge_slots,
                       size_t stage_bytes, int warps) {
  return ring_smem(table_rows, repk_log2, repv_log2, d, outl, stages, merge_slots, stage_bytes, warps).total;
}

}  // namespace attn
}  // namespace hqmq
