/*
 * uccl_device.cuh -- one-sided operations callable from inside user kernels.
 *
 * Counterpart of the reference's device RMA header (src/rma/rma_device.hpp:47-387): a POD window
 * descriptor that is passed to kernels by value, put / get as grid-stride copies to or from a
 * peer's mapped memory, signals as monotonic 64-bit counters (one per receiver and sender),
 * bounded waits.  On NVLink the accesses are ordinary loads and stores on peer-mapped addresses;
 * signals use red.release.sys / ld.acquire.sys so that data written before a signal is visible
 * to the peer that observed it.
 *
 * Obtain the descriptor on the host with ucclWindowGetDeviceHandle().
 */
#ifndef UCCL_DEVICE_CUH_
#define UCCL_DEVICE_CUH_

#include <cuda_runtime.h>
#include <stdint.h>

#include "uccl.h"

typedef struct {
  char* localBuff;
  char* remotePtrs[UCCL_MAX_LOCAL_RANKS];          /* peers' window memory, mapped here        */
  size_t size;
  int nRanks;
  int myRank;
  unsigned long long* localSignals;                /* [nRanks], slot p counts signals from p   */
  unsigned long long* remoteSignals[UCCL_MAX_LOCAL_RANKS]; /* peers' signal arrays, mapped here */
  unsigned long long timeoutNs;                    /* budget of deviceWaitSignal               */
} ucclDeviceWindow;

#ifdef __cplusplus
extern "C" {
#endif
ucclResult_t ucclWindowGetDeviceHandle(ucclWindow_t win, ucclDeviceWindow* deviceWin);
#ifdef __cplusplus
}
#endif

#if defined(__CUDACC__)

namespace uccl_device {

__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void signal_add(unsigned long long* p, unsigned long long v) {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long signal_load(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

/* grid-stride byte copy; 16-byte vectors when both sides allow it */
__device__ __forceinline__ void copy_bytes(char* dst, const char* src, size_t bytes) {
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
    const size_t nv = bytes >> 4;
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    for (size_t i = tid; i < nv; i += nth) d[i] = s[i];
    for (size_t i = (nv << 4) + tid; i < bytes; i += nth) dst[i] = src[i];
  } else {
    for (size_t i = tid; i < bytes; i += nth) dst[i] = src[i];
  }
}

}  // namespace uccl_device

/* ---- put / get ---------------------------------------------------------------------------- */
__device__ __forceinline__ void devicePut(const ucclDeviceWindow& w, int peer, size_t peerOffset, const void* local,
                                          size_t bytes) {
  uccl_device::copy_bytes(w.remotePtrs[peer] + peerOffset, static_cast<const char*>(local), bytes);
}
template <typename T>
__device__ __forceinline__ void devicePutElements(const ucclDeviceWindow& w, int peer, size_t peerElemOffset,
                                                  const T* local, size_t count) {
  devicePut(w, peer, peerElemOffset * sizeof(T), local, count * sizeof(T));
}
__device__ __forceinline__ void deviceGet(const ucclDeviceWindow& w, int peer, size_t peerOffset, void* local,
                                          size_t bytes) {
  uccl_device::copy_bytes(static_cast<char*>(local), w.remotePtrs[peer] + peerOffset, bytes);
}
template <typename T>
__device__ __forceinline__ void deviceGetElements(const ucclDeviceWindow& w, int peer, size_t peerElemOffset, T* local,
                                                  size_t count) {
  deviceGet(w, peer, peerElemOffset * sizeof(T), local, count * sizeof(T));
}

/* ---- signals ------------------------------------------------------------------------------ */
/* Raise the counter that `peer` keeps for this rank.  Call from ONE thread. */
__device__ __forceinline__ void deviceSignal(const ucclDeviceWindow& w, int peer) {
  uccl_device::signal_add(w.remoteSignals[peer] + w.myRank, 1ull);
}
/* Put, then signal once the whole CTA's part has been written.  All threads of the CTA call;
 * every CTA of the grid raises the signal once, so the receiver expects gridDim.x per call --
 * launch with one CTA when a single increment per put is wanted. */
__device__ __forceinline__ void devicePutSignal(const ucclDeviceWindow& w, int peer, size_t peerOffset,
                                                const void* local, size_t bytes) {
  devicePut(w, peer, peerOffset, local, bytes);
  __syncthreads();
  if (threadIdx.x == 0) deviceSignal(w, peer);
}
/* Get, then bump the local counter of `peer` (completion marker for this rank's own waits). */
__device__ __forceinline__ void deviceGetSignal(const ucclDeviceWindow& w, int peer, size_t peerOffset, void* local,
                                                size_t bytes) {
  deviceGet(w, peer, peerOffset, local, bytes);
  __syncthreads();
  if (threadIdx.x == 0) uccl_device::signal_add(w.localSignals + peer, 1ull);
}
/* Wait until `peer` has signalled at least `expected` times in total.  Bounded: returns false
 * when the window's time budget ran out.  Call from one thread (or use the cooperative form). */
__device__ __forceinline__ bool deviceWaitSignal(const ucclDeviceWindow& w, int peer, unsigned long long expected) {
  const unsigned long long* p = w.localSignals + peer;
  if (uccl_device::signal_load(p) >= expected) return true;
  const unsigned long long t0 = uccl_device::globaltimer();
  unsigned int spins = 0;
  while (uccl_device::signal_load(p) < expected) {
    if ((++spins & 63u) == 0 && w.timeoutNs && uccl_device::globaltimer() - t0 > w.timeoutNs) return false;
  }
  return true;
}
/* Thread 0 waits, the whole CTA learns the outcome. */
__device__ __forceinline__ bool deviceWaitSignalCooperative(const ucclDeviceWindow& w, int peer,
                                                            unsigned long long expected) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = deviceWaitSignal(w, peer, expected) ? 1 : 0;
  __syncthreads();
  const bool r = ok != 0;
  __syncthreads();
  return r;
}
/* Wait for several peers at once. */
__device__ __forceinline__ bool deviceWaitSignalMulti(const ucclDeviceWindow& w, const int* peers,
                                                      const unsigned long long* expected, int n) {
  bool all = true;
  for (int i = 0; i < n; ++i) all = deviceWaitSignal(w, peers[i], expected[i]) && all;
  return all;
}
/* local[i] = local[i] + remote[i] for `count` floats: fused pull + reduce. */
__device__ __forceinline__ void deviceGetReduceF32(const ucclDeviceWindow& w, int peer, size_t peerElemOffset,
                                                   float* local, size_t count) {
  const float* remote = reinterpret_cast<const float*>(w.remotePtrs[peer]) + peerElemOffset;
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = tid; i < count; i += nth) local[i] += remote[i];
}

#endif /* __CUDACC__ */
#endif /* UCCL_DEVICE_CUH_ */
