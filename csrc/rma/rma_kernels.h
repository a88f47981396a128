// Small kernels behind the host-side one-sided API (see rma_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../kernels/device_comm.h"

namespace uccl {

// dst[0..bytes) = src[0..bytes) (peer or local memory), then *signal += 1 with release order.
// signal may be nullptr (plain put/get).
cudaError_t launchRmaCopySignal(char* dst, const char* src, size_t bytes, uint64_t* signal, uint32_t* scratchCounter,
                                cudaStream_t stream);
// *signal += 1 after everything earlier in the stream.
cudaError_t launchRmaSignal(uint64_t* signal, cudaStream_t stream);
struct RmaWaitArgs {
  DevComm dc;
  int n;
  const uint64_t* signals[8];
  uint64_t expected[8];
  int peers[8];
};
cudaError_t launchRmaWait(const RmaWaitArgs& a, cudaStream_t stream);

}  // namespace uccl
