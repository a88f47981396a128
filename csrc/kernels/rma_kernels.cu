// Kernels of the host-side one-sided API: copy (+ signal), signal, bounded wait.
//
// The reference issues queue.memcpy followed by a single_task that fences and increments the
// counter (src/rma/rma.cc:338-360, :416-425) and a single_task that spins up to 1e8 times per
// descriptor and gives up silently (src/rma/rma.cc:542-559).  Here small and medium transfers are
// one kernel that copies and then signals (one launch instead of two), and a wait that runs out
// of time records the reason in the communicator's status words.
#include "../rma/rma_kernels.h"
#include "coll_device.cuh"

namespace uccl {
namespace dev {

__global__ void __launch_bounds__(kThreads) rma_copy_signal_kernel(char* dst, const char* src, size_t bytes,
                                                                   uint64_t* signal, uint32_t* counter) {
  size_t off, len;
  {
    size_t o, l;
    split(bytes >> 4, gridDim.x, blockIdx.x, &o, &l);
    off = o << 4;
    len = l << 4;
    if (blockIdx.x == gridDim.x - 1) len += bytes & 15;
  }
  block_copy(dst + off, src + off, len);
  if (!signal) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    ptx::fence_sys();
    // the last CTA to finish raises the signal; the counter returns to zero for the next call
    const uint32_t prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x - 1) {
      *counter = 0;
      ptx::fence_sys();
      ptx::red_release_sys_add_u64(signal, 1ull);
    }
  }
}

__global__ void rma_signal_kernel(uint64_t* signal) {
  ptx::fence_sys();
  ptx::red_release_sys_add_u64(signal, 1ull);
}

__global__ void rma_wait_kernel(const __grid_constant__ RmaWaitArgs a) {
  const int i = threadIdx.x;
  if (i < a.n) wait_u64(a.signals[i], a.expected[i], a.dc, DEV_TIMEOUT_SIGNAL, a.peers[i], static_cast<uint32_t>(a.expected[i]));
}

}  // namespace dev

cudaError_t launchRmaCopySignal(char* dst, const char* src, size_t bytes, uint64_t* signal, uint32_t* counter,
                                cudaStream_t stream) {
  int blocks = static_cast<int>((bytes + (128u << 10) - 1) / (128u << 10));
  if (blocks < 1) blocks = 1;
  if (blocks > 32) blocks = 32;
  dev::rma_copy_signal_kernel<<<blocks, dev::kThreads, 0, stream>>>(dst, src, bytes, signal, counter);
  return cudaGetLastError();
}
cudaError_t launchRmaSignal(uint64_t* signal, cudaStream_t stream) {
  dev::rma_signal_kernel<<<1, 1, 0, stream>>>(signal);
  return cudaGetLastError();
}
cudaError_t launchRmaWait(const RmaWaitArgs& a, cudaStream_t stream) {
  dev::rma_wait_kernel<<<1, 32, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace uccl
