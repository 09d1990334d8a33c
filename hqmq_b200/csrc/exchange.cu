// Exchange of sequence-split attention partials between GPUs by direct stores over NVLink.
//
// When one long context is split by sequence over N GPUs, every GPU ends a decode step with one block of
// un-normalised partial results (o[d], m, l per query head: 17 KB at 32 heads x d 128) that every other GPU
// needs before it can merge.  An all_gather does that with a collective launch on every rank; here each rank
// instead WRITES its block into slot `rank` of every peer's receive buffer (peer-mapped pointers, plain
// vectorised stores), then publishes a per-step epoch word with a system-scope release store.  The consumer
// polls only its OWN memory, with a bounded number of polls; a wait that runs out records the missing ranks
// in a status word and returns, so the context stays usable and the host can report the failure.
//
// No load ever targets a peer's memory, nothing is multicast, and no kernel of one GPU waits for another
// kernel of the SAME GPU: the producer of every flag a kernel polls runs on a different device.
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/hqmq_b200.h"
#include "common.cuh"

#include <cstring>

namespace hqmq {
namespace {

constexpr uint32_t kDefaultPolls = 1u << 19;     // a poll is a system-scope load (~1 us) + 100 ns of sleep: gives up after roughly a second

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One CTA per destination rank (this rank's own receive buffer included).
__global__ void __launch_bounds__(256)
push_kernel(hqmq_exchange x, const float* __restrict__ local, uint32_t epoch) {
  const int p = blockIdx.x;
  const int par = (int)(epoch & 1u);
  float* dst = x.recv[p] + ((int64_t)par * x.world + x.rank) * x.block_floats;
  const int64_t n4 = x.block_floats >> 2;
  const float4* s4 = reinterpret_cast<const float4*>(local);
  float4* d4 = reinterpret_cast<float4*>(dst);
  for (int64_t i = threadIdx.x; i < n4; i += blockDim.x) d4[i] = s4[i];
  for (int64_t i = (n4 << 2) + threadIdx.x; i < x.block_floats; i += blockDim.x) dst[i] = local[i];
  __threadfence_system();          // every thread's stores are visible system-wide before the epoch word is
  __syncthreads();
  if (threadIdx.x == 0) st_release_sys(x.flags[p] + par * x.world + x.rank, epoch);
}

// One CTA; thread r waits for rank r's epoch word in this GPU's own memory.
__global__ void __launch_bounds__(32)
wait_kernel(hqmq_exchange x, uint32_t epoch, uint32_t max_polls, uint32_t* __restrict__ status) {
  const int r = threadIdx.x;
  const int par = (int)(epoch & 1u);
  bool missing = false;
  if (r < x.world) {
    const uint32_t* f = x.flags[x.rank] + par * x.world + r;
    uint32_t polls = 0;
    while (ld_acquire_sys(f) != epoch) {
      if (++polls >= max_polls) { missing = true; break; }
      __nanosleep(100);
    }
  }
  const uint32_t miss = __ballot_sync(0xffffffffu, missing);
  if (r == 0 && miss) atomicOr(status, miss);     // bit r = rank r's block of this step never arrived
}

// Push, bounded wait and merge of one step in ONE launch.  CTAs [0, world) store this rank's block into the ranks'
// receive buffers and publish the epoch (as push_kernel does); CTA world + r waits, with the bound of wait_kernel, for
// all ranks' epoch words in this GPU's own memory and then merges row r of their blocks.  The CTAs that wait depend
// on other GPUs' stores only, never on a CTA of this launch or of another kernel of this GPU, and the grid
// (world + rows CTAs) is far below what the GPU holds resident, so the pushing CTAs always get to run.  The received
// blocks were written by other GPUs while this kernel may already be running: they are read past the L1 (ld.global.cg).
__global__ void __launch_bounds__(128)
step_kernel(hqmq_exchange x, const float* __restrict__ local, uint32_t epoch, uint32_t max_polls, uint32_t* __restrict__ status,
            int rows, int d, int out_dtype, void* __restrict__ out) {
  const int par = (int)(epoch & 1u);
  if ((int)blockIdx.x < x.world) {
    const int p = blockIdx.x;
    float* dst = x.recv[p] + ((int64_t)par * x.world + x.rank) * x.block_floats;
    const int64_t n4 = x.block_floats >> 2;
    const float4* s4 = reinterpret_cast<const float4*>(local);
    float4* d4 = reinterpret_cast<float4*>(dst);
    for (int64_t i = threadIdx.x; i < n4; i += blockDim.x) d4[i] = s4[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(x.flags[p] + par * x.world + x.rank, epoch);
    return;
  }
  const int row = (int)blockIdx.x - x.world;
  if (row >= rows) return;
  __shared__ float s_m[HQMQ_EXCHANGE_MAX_RANKS], s_l[HQMQ_EXCHANGE_MAX_RANKS];
  __shared__ uint32_t s_miss;
  if (threadIdx.x == 0) s_miss = 0u;
  __syncthreads();
  const float* blocks = x.recv[x.rank] + (int64_t)par * x.world * x.block_floats;
  if ((int)threadIdx.x < x.world) {
    const int r = threadIdx.x;
    const uint32_t* f = x.flags[x.rank] + par * x.world + r;
    uint32_t polls = 0;
    bool missing = false;
    while (ld_acquire_sys(f) != epoch) {
      if (++polls >= max_polls) { missing = true; break; }
      __nanosleep(100);
    }
    if (missing) atomicOr(&s_miss, 1u << r);
    const float* pr = blocks + (int64_t)r * x.block_floats + (int64_t)row * (d + 2);
    s_m[r] = __ldcg(pr + d);
    s_l[r] = __ldcg(pr + d + 1);
  }
  __syncthreads();
  if (s_miss) {                                   // some rank's block of this step never arrived: report, write nothing valid
    if (threadIdx.x == 0 && row == 0) atomicOr(status, s_miss);
  }
  float m_star = -INFINITY;
  for (int r = 0; r < x.world; ++r) m_star = fmaxf(m_star, s_m[r]);
  const float m_use = m_star == -INFINITY ? 0.f : m_star;
  // (the denominator is summed in the order hqmq_combine_partials uses -- one term per lane, a butterfly over the
  //  warp -- so that this launch and the three-call form give the same bits)
  __shared__ float s_lstar;
  if (threadIdx.x < 32) {
    float l_loc = (int)threadIdx.x < x.world ? s_l[threadIdx.x] * exp2f(s_m[threadIdx.x] - m_use) : 0.f;
    for (int o = 16; o > 0; o >>= 1) l_loc += __shfl_xor_sync(0xffffffffu, l_loc, o);
    if (threadIdx.x == 0) s_lstar = l_loc;
  }
  __syncthreads();
  const float l_star = s_lstar;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < x.world; ++r) {
      const float w = exp2f(s_m[r] - m_use);
      if (w != 0.f) acc += __ldcg(blocks + (int64_t)r * x.block_floats + (int64_t)row * (d + 2) + c) * w;
    }
    if (s_miss) acc = NAN;
    store_float(out, (int64_t)row * d + c, l_star > 0.f || s_miss ? acc / l_star : 0.f, out_dtype);
  }
}

int validate(const hqmq_exchange* x) {
  if (!x || x->struct_size != sizeof(hqmq_exchange)) return HQMQ_ERR_ARG;
  if (x->world < 1 || x->world > HQMQ_EXCHANGE_MAX_RANKS || x->rank < 0 || x->rank >= x->world) return HQMQ_ERR_ARG;
  if (x->block_floats < 1) return HQMQ_ERR_SHAPE;
  for (int p = 0; p < x->world; ++p) {
    if (!x->recv[p] || !x->flags[p]) return HQMQ_ERR_ARG;
    if (((uintptr_t)x->recv[p] & 15) || ((uintptr_t)x->flags[p] & 3)) return HQMQ_ERR_ALIGN;
  }
  if (x->block_floats % 4) return HQMQ_ERR_ALIGN;   // every slot starts on a 16-byte boundary
  return HQMQ_OK;
}

}  // namespace
}  // namespace hqmq
using namespace hqmq;

extern "C" size_t hqmq_exchange_recv_bytes(int world, int64_t block_floats) {
  if (world < 1 || world > HQMQ_EXCHANGE_MAX_RANKS || block_floats < 1) return 0;
  return (size_t)2 * world * block_floats * sizeof(float);
}

extern "C" size_t hqmq_exchange_flag_bytes(int world) {
  if (world < 1 || world > HQMQ_EXCHANGE_MAX_RANKS) return 0;
  return (size_t)2 * world * sizeof(uint32_t);
}

extern "C" int hqmq_exchange_enable_peer(int peer_device) {
  int cur = -1, can = 0;
  HQMQ_CHECK_CUDA(cudaGetDevice(&cur));
  if (peer_device == cur) return HQMQ_OK;
  if (cudaDeviceCanAccessPeer(&can, cur, peer_device) != cudaSuccess) { cudaGetLastError(); return HQMQ_ERR_ARG; }
  if (!can) return HQMQ_ERR_UNSUPPORTED;
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return HQMQ_OK; }   // clear the sticky-free error
  return e == cudaSuccess ? HQMQ_OK : HQMQ_ERR_CUDA;
}

// ---- mapping a peer process's receive buffer ---------------------------------------------------------------
// An IPC mapping is made "into the current device's address space": a mapping opened with the buffer's OWN
// device current (what a tensor-sharing layer does, because it wants to use the tensor on that device) is not
// reachable by kernels of another device of the same process, peer access or not.  So the buffer is opened
// here with the ACCESSING device current and cudaIpcMemLazyEnablePeerAccess, the pattern collective libraries use.
extern "C" int hqmq_exchange_ipc_export(const void* ptr, unsigned char* handle64, int64_t* offset) {
  if (!ptr || !handle64 || !offset) return HQMQ_ERR_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == HQMQ_IPC_HANDLE_BYTES, "IPC handle size");
  // the handle names the whole allocation the address lies in; its start comes from the driver
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
      q != cudaDriverEntryPointSuccess) { cudaGetLastError(); return HQMQ_ERR_CUDA; }
  CUdeviceptr base = 0; size_t size = 0;
  if (reinterpret_cast<RangeFn>(fn)(&base, &size, (CUdeviceptr)(uintptr_t)ptr) != CUDA_SUCCESS || !base) return HQMQ_ERR_ARG;
  cudaIpcMemHandle_t h;
  HQMQ_CHECK_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base)));
  memcpy(handle64, &h, sizeof(h));
  *offset = (int64_t)((uintptr_t)ptr - (uintptr_t)base);
  return HQMQ_OK;
}

extern "C" int hqmq_exchange_ipc_open(const unsigned char* handle64, void** base_out) {
  if (!handle64 || !base_out) return HQMQ_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* base = nullptr;
  if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || !base) { cudaGetLastError(); return HQMQ_ERR_CUDA; }
  *base_out = base;
  return HQMQ_OK;
}

extern "C" int hqmq_exchange_ipc_close(void* base) {
  if (!base) return HQMQ_ERR_ARG;
  HQMQ_CHECK_CUDA(cudaIpcCloseMemHandle(base));
  return HQMQ_OK;
}

extern "C" int hqmq_exchange_verify(const hqmq_exchange* x) {
  int rc = validate(x);
  if (rc) return rc;
  int cur = -1;
  HQMQ_CHECK_CUDA(cudaGetDevice(&cur));
  for (int p = 0; p < x->world; ++p) {
    const void* ptrs[2] = {x->recv[p], x->flags[p]};
    for (const void* q : ptrs) {
      // a host address or an unmapped one would fault in the kernel: refuse it here
      cudaPointerAttributes at;
      if (cudaPointerGetAttributes(&at, q) != cudaSuccess || at.type != cudaMemoryTypeDevice) { cudaGetLastError(); return HQMQ_ERR_ARG; }
      if (p == x->rank && at.device != cur) return HQMQ_ERR_ARG;    // the own buffers live on the current device
      if (at.device != cur) {
        rc = hqmq_exchange_enable_peer(at.device);
        if (rc) return rc;
      }
    }
  }
  return HQMQ_OK;
}

extern "C" int hqmq_exchange_push(const hqmq_exchange* x, const float* local, uint32_t epoch, void* stream) {
  int rc = validate(x);
  if (rc) return rc;
  if (!local || epoch == 0) return HQMQ_ERR_ARG;
  if ((uintptr_t)local & 15) return HQMQ_ERR_ALIGN;
  push_kernel<<<x->world, 256, 0, (cudaStream_t)stream>>>(*x, local, epoch);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

extern "C" int hqmq_exchange_wait(const hqmq_exchange* x, uint32_t epoch, uint32_t max_polls, uint32_t* status,
                                  void* stream) {
  int rc = validate(x);
  if (rc) return rc;
  if (!status || epoch == 0) return HQMQ_ERR_ARG;
  wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(*x, epoch, max_polls ? max_polls : kDefaultPolls, status);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}

extern "C" int hqmq_exchange_step(const hqmq_exchange* x, const float* local, uint32_t epoch, uint32_t max_polls,
                                  uint32_t* status, int64_t rows, int d, int out_dtype, void* out, void* stream) {
  int rc = validate(x);
  if (rc) return rc;
  if (!local || !status || !out || epoch == 0) return HQMQ_ERR_ARG;
  if ((uintptr_t)local & 15) return HQMQ_ERR_ALIGN;
  if (rows < 1 || d < 1 || rows * (int64_t)(d + 2) != x->block_floats) return HQMQ_ERR_SHAPE;
  if (!is_float_dtype(out_dtype)) return HQMQ_ERR_DTYPE;
  if (rows + x->world > 148 * 8) return HQMQ_ERR_UNSUPPORTED;   // every CTA of the launch resident at once, so that the pushing
                                                                // CTAs never queue behind waiting ones (larger problems: push, wait, merge)
  step_kernel<<<(unsigned)(x->world + rows), 128, 0, (cudaStream_t)stream>>>(*x, local, epoch, max_polls ? max_polls : kDefaultPolls,
                                                                            status, (int)rows, d, out_dtype, out);
  HQMQ_LAUNCH_CHECK();
  return HQMQ_OK;
}
