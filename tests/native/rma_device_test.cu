// Test-only kernels that call the device-side one-sided API (include/uccl_device.cuh) from
// inside a kernel, the way a user kernel would.  Built into tests/native/libuccl_devtest.so and
// driven through ctypes by tests/rank_worker.py (case "rma_device").
//
// The reference declares the same calls as SYCL inlines (src/rma/rma_device.hpp:84-357) and has
// no test for them.
//
// Compiled with the header's checked mode on: every access of the tests below passes through the
// bounds test, and ucclDevTestCheckRead returns the record of the ones it refused.
#define UCCL_DEVICE_CHECKS 1
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "uccl_device.cuh"

namespace {

// One CTA: copy `bytes` into the peer's window at `peerOff`, then raise the peer's counter once.
template <typename W>
__global__ void put_signal_kernel(const W w, int peer, size_t peerOff, const char* local, size_t bytes) {
  devicePutSignal(w, peer, peerOff, local, bytes);
}

// One CTA: wait for `expected` signals from `peer` (cooperative form), report the outcome, then
// combine `count` elements of the peer's window with local data.
template <typename T, typename W>
__global__ void wait_reduce_kernel(const W w, int peer, unsigned long long expected, const T* local, T* result,
                                   size_t count, size_t peerByteOff, int* okOut) {
  const bool ok = deviceWaitSignalCooperative(w, peer, expected);
  if (threadIdx.x == 0) *okOut = ok ? 1 : 0;
  if (!ok) return;
  if (count) deviceGetReduce<T, ucclDeviceSum>(w, local, result, count, peer, peerByteOff);
}

// One CTA: wait for several peers at once (single thread), then pull `bytes` from the first peer
// and count the pull on the local counter of that peer.
template <typename W>
__global__ void wait_multi_get_kernel(const W w, const int* peers, const unsigned long long* expected, int n,
                                      size_t peerOff, char* local, size_t bytes, int* okOut) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = deviceWaitSignalMulti(w, peers, expected, n) ? 1 : 0;
    *okOut = ok;
  }
  __syncthreads();
  if (!ok) return;
  deviceGetSignal(w, peers[0], peerOff, local, bytes);
}

template <typename W>
__global__ void put_elements_kernel(const W w, int peer, size_t elemOff, const float* local, size_t count) {
  devicePutElements<float>(w, peer, elemOff, local, count);
  __syncthreads();
  if (threadIdx.x == 0) deviceSignal(w, peer);
}

template <typename W>
__global__ void get_elements_kernel(const W w, int peer, size_t elemOff, float* local, size_t count) {
  deviceGetElements<float>(w, peer, elemOff, local, count);
}

int check(cudaError_t e) { return e == cudaSuccess ? 0 : 1000 + static_cast<int>(e); }

template <typename W>
int getWindow(void* win, W* out);
template <>
int getWindow<ucclDeviceWindow>(void* win, ucclDeviceWindow* out) {
  return ucclWindowGetDeviceHandle(static_cast<ucclWindow_t>(win), out) == ucclSuccess ? 0 : 1;
}
template <>
int getWindow<ucclDeviceWindowDyn>(void* win, ucclDeviceWindowDyn* out) {
  return ucclWindowGetDeviceHandleDyn(static_cast<ucclWindow_t>(win), out) == ucclSuccess ? 0 : 1;
}

template <typename W>
int putSignal(void* win, int peer, size_t peerOff, const void* local, size_t bytes, void* stream) {
  W w;
  if (getWindow(win, &w)) return 1;
  put_signal_kernel<W><<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(w, peer, peerOff, static_cast<const char*>(local), bytes);
  return check(cudaGetLastError());
}

template <typename W>
int waitReduce(void* win, int peer, unsigned long long expected, int dtype, const void* local, void* result,
               size_t count, size_t peerByteOff, int* okOut, void* stream) {
  W w;
  if (getWindow(win, &w)) return 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case ucclFloat32:
      wait_reduce_kernel<float, W><<<1, 256, 0, s>>>(w, peer, expected, static_cast<const float*>(local),
                                                     static_cast<float*>(result), count, peerByteOff, okOut);
      break;
    case ucclBfloat16:
      wait_reduce_kernel<__nv_bfloat16, W><<<1, 256, 0, s>>>(w, peer, expected, static_cast<const __nv_bfloat16*>(local),
                                                             static_cast<__nv_bfloat16*>(result), count, peerByteOff, okOut);
      break;
    case ucclFloat16:
      wait_reduce_kernel<__half, W><<<1, 256, 0, s>>>(w, peer, expected, static_cast<const __half*>(local),
                                                      static_cast<__half*>(result), count, peerByteOff, okOut);
      break;
    default: return 2;
  }
  return check(cudaGetLastError());
}

}  // namespace

extern "C" {

// out[4]: count of refused accesses, (kind << 32 | peer), offset, bytes of the first; clears the record
int ucclDevTestCheckRead(unsigned long long* out) { return check(ucclDeviceCheckRead(out)); }

// dyn != 0 selects the pointer-table descriptor (ucclDeviceWindowDyn).
int ucclDevTestPutSignal(void* win, int dyn, int peer, size_t peerOff, const void* local, size_t bytes, void* stream) {
  return dyn ? putSignal<ucclDeviceWindowDyn>(win, peer, peerOff, local, bytes, stream)
             : putSignal<ucclDeviceWindow>(win, peer, peerOff, local, bytes, stream);
}

int ucclDevTestWaitReduce(void* win, int dyn, int peer, unsigned long long expected, int dtype, const void* local,
                          void* result, size_t count, size_t peerByteOff, int* okOut, void* stream) {
  return dyn ? waitReduce<ucclDeviceWindowDyn>(win, peer, expected, dtype, local, result, count, peerByteOff, okOut, stream)
             : waitReduce<ucclDeviceWindow>(win, peer, expected, dtype, local, result, count, peerByteOff, okOut, stream);
}

// peers / expected are device arrays of n entries
int ucclDevTestWaitMultiGet(void* win, const int* peers, const unsigned long long* expected, int n, size_t peerOff,
                            void* local, size_t bytes, int* okOut, void* stream) {
  ucclDeviceWindow w;
  if (getWindow(win, &w)) return 1;
  wait_multi_get_kernel<ucclDeviceWindow><<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, peers, expected, n, peerOff, static_cast<char*>(local), bytes, okOut);
  return check(cudaGetLastError());
}

int ucclDevTestPutElements(void* win, int peer, size_t elemOff, const void* local, size_t count, void* stream) {
  ucclDeviceWindow w;
  if (getWindow(win, &w)) return 1;
  put_elements_kernel<ucclDeviceWindow><<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, peer, elemOff, static_cast<const float*>(local), count);
  return check(cudaGetLastError());
}

int ucclDevTestGetElements(void* win, int peer, size_t elemOff, void* local, size_t count, void* stream) {
  ucclDeviceWindow w;
  if (getWindow(win, &w)) return 1;
  get_elements_kernel<ucclDeviceWindow><<<4, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, peer, elemOff, static_cast<float*>(local), count);
  return check(cudaGetLastError());
}

// A descriptor assembled by hand with makeDeviceWindow() must equal the library's own.
int ucclDevTestMakeWindow(void* win) {
  ucclDeviceWindow a;
  if (getWindow(win, &a)) return 1;
  void* rp[UCCL_MAX_LOCAL_RANKS];
  unsigned long long* rs[UCCL_MAX_LOCAL_RANKS];
  for (int p = 0; p < a.nRanks; ++p) {
    rp[p] = a.remotePtrs[p];
    rs[p] = a.remoteSignals[p];
  }
  const ucclDeviceWindow b = makeDeviceWindow(a.localBuff, rp, a.localSignals, rs, a.size, a.nRanks, a.myRank, a.timeoutNs);
  if (b.localBuff != a.localBuff || b.size != a.size || b.nRanks != a.nRanks || b.myRank != a.myRank ||
      b.localSignals != a.localSignals || b.timeoutNs != a.timeoutNs)
    return 2;
  for (int p = 0; p < a.nRanks; ++p)
    if (b.remotePtrs[p] != a.remotePtrs[p] || b.remoteSignals[p] != a.remoteSignals[p]) return 3;
  return 0;
}

}  // extern "C"
