/*
 * uccl_device.cuh -- one-sided operations callable from inside user kernels.
 *
 * Counterpart of the reference's device RMA header (src/rma/rma_device.hpp:47-387): a window
 * descriptor that is passed to kernels by value, put / get as grid-stride copies to or from a
 * peer's mapped memory, signals as monotonic 64-bit counters (one per receiver and sender),
 * bounded waits, and a fused pull + reduce.  On NVLink the accesses are ordinary loads and stores
 * on peer-mapped addresses; signals use red.release.sys / ld.acquire.sys so that data written
 * before a signal is visible to the peer that observed it.
 *
 * Two descriptor forms, as in the reference (rma_device.hpp:47-70):
 *   ucclDeviceWindow     fixed-size tables inside the struct (UCCL_MAX_LOCAL_RANKS peers),
 *   ucclDeviceWindowDyn  tables behind device pointers, for code that keeps descriptors small.
 * Every function below is a template on the descriptor type and takes either form.
 *
 * Obtain a descriptor on the host with ucclWindowGetDeviceHandle() / ucclWindowGetDeviceHandleDyn(),
 * or assemble one from raw tables with makeDeviceWindow() (rma_device.hpp:365).
 *
 * Checked build: compile the including file with -DUCCL_DEVICE_CHECKS and every put / get /
 * get-reduce / signal first tests its peer index and byte range against the descriptor
 * (peer < nRanks, offset + bytes <= size).  An access that fails the test is left out and
 * recorded (first one wins: kind, peer, offset, bytes) in a device variable of the including
 * translation unit, which ucclDeviceCheckRead() copies to the host.  The reference has no bounds
 * checks on this path (rma_device.hpp:86-127 index remotePtrs[peer] + offset directly).
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

/* Same content with the two per-peer tables in device memory (owned by the window). */
typedef struct {
  char* localBuff;
  char** remotePtrs;                               /* device array [nRanks]                    */
  size_t size;
  int nRanks;
  int myRank;
  unsigned long long* localSignals;
  unsigned long long** remoteSignals;              /* device array [nRanks]                    */
  unsigned long long timeoutNs;
} ucclDeviceWindowDyn;

#ifdef __cplusplus
extern "C" {
#endif
ucclResult_t ucclWindowGetDeviceHandle(ucclWindow_t win, ucclDeviceWindow* deviceWin);
/* The tables live in device memory that the window owns until ucclCommWindowDeregister. */
ucclResult_t ucclWindowGetDeviceHandleDyn(ucclWindow_t win, ucclDeviceWindowDyn* deviceWin);
#ifdef __cplusplus
}

/* Host helper: a by-value descriptor from raw tables (at most UCCL_MAX_LOCAL_RANKS entries are
 * taken).  timeoutNs = 0 selects the default budget of ten seconds. */
static inline ucclDeviceWindow makeDeviceWindow(void* localBuff, void* const* remotePtrs,
                                                unsigned long long* localSignals,
                                                unsigned long long* const* remoteSignals, size_t size, int nRanks,
                                                int myRank, unsigned long long timeoutNs = 0) {
  ucclDeviceWindow w = {};
  w.localBuff = static_cast<char*>(localBuff);
  w.size = size;
  w.nRanks = nRanks;
  w.myRank = myRank;
  w.localSignals = localSignals;
  w.timeoutNs = timeoutNs;
  for (int r = 0; r < nRanks && r < UCCL_MAX_LOCAL_RANKS; ++r) {
    w.remotePtrs[r] = static_cast<char*>(remotePtrs[r]);
    w.remoteSignals[r] = remoteSignals[r];
  }
  return w;
}
#endif

#if defined(__CUDACC__)

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace uccl_device {

constexpr unsigned long long kDefaultWaitNs = 10000000000ull;  /* a wait never runs without a limit */

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

#ifdef UCCL_DEVICE_CHECKS
/* [0] = number of refused accesses, [1] = kind (1 put, 2 get, 3 get-reduce, 4 signal) << 32 | peer,
 * [2] = byte offset, [3] = bytes of the first refused access */
static __device__ unsigned long long g_check_record[4];
template <typename W>
__device__ __forceinline__ bool access_ok(const W& w, int kind, int peer, size_t off, size_t bytes) {
  if (peer >= 0 && peer < w.nRanks && off <= w.size && bytes <= w.size - off) return true;
  if (blockIdx.x == 0 && threadIdx.x == 0) {  /* the grid makes the call together: one record per call */
    if (atomicAdd(&g_check_record[0], 1ull) == 0ull) {
      g_check_record[1] = (static_cast<unsigned long long>(kind) << 32) | static_cast<unsigned int>(peer);
      g_check_record[2] = off;
      g_check_record[3] = bytes;
    }
  }
  return false;
}
#define UCCL_DEVICE_ACCESS_OK(w, kind, peer, off, bytes) uccl_device::access_ok(w, kind, peer, off, bytes)
#else
#define UCCL_DEVICE_ACCESS_OK(w, kind, peer, off, bytes) true
#endif

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

/* element <-> float, so that 16-bit types are combined in fp32 (the reference's ReduceSum adds in
 * the element type, src/device/reduce_kernel.hpp:17-20) */
template <typename T> __device__ __forceinline__ float to_float(T v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half(v); }

}  // namespace uccl_device

/* Reduction functors for deviceGetReduce; operands arrive as fp32. */
struct ucclDeviceSum {
  __device__ __forceinline__ float operator()(float a, float b) const { return a + b; }
};
struct ucclDeviceMax {
  __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); }
};
struct ucclDeviceMin {
  __device__ __forceinline__ float operator()(float a, float b) const { return fminf(a, b); }
};

/* ---- put / get ---------------------------------------------------------------------------- */
/* The whole grid takes part: every thread copies its share.  */
template <typename W>
__device__ __forceinline__ void devicePut(const W& w, int peer, size_t peerOffset, const void* local, size_t bytes) {
  if (!UCCL_DEVICE_ACCESS_OK(w, 1, peer, peerOffset, bytes)) return;
  uccl_device::copy_bytes(w.remotePtrs[peer] + peerOffset, static_cast<const char*>(local), bytes);
}
template <typename T, typename W>
__device__ __forceinline__ void devicePutElements(const W& w, int peer, size_t peerElemOffset, const T* local,
                                                  size_t count) {
  devicePut(w, peer, peerElemOffset * sizeof(T), local, count * sizeof(T));
}
template <typename W>
__device__ __forceinline__ void deviceGet(const W& w, int peer, size_t peerOffset, void* local, size_t bytes) {
  if (!UCCL_DEVICE_ACCESS_OK(w, 2, peer, peerOffset, bytes)) return;
  uccl_device::copy_bytes(static_cast<char*>(local), w.remotePtrs[peer] + peerOffset, bytes);
}
template <typename T, typename W>
__device__ __forceinline__ void deviceGetElements(const W& w, int peer, size_t peerElemOffset, T* local, size_t count) {
  deviceGet(w, peer, peerElemOffset * sizeof(T), local, count * sizeof(T));
}

/* ---- signals ------------------------------------------------------------------------------ */
/* Raise the counter that `peer` keeps for this rank.  Call from ONE thread. */
template <typename W>
__device__ __forceinline__ void deviceSignal(const W& w, int peer) {
  if (!UCCL_DEVICE_ACCESS_OK(w, 4, peer, 0, 0)) return;
  uccl_device::signal_add(w.remoteSignals[peer] + w.myRank, 1ull);
}
/* Put, then signal once the whole CTA's part has been written.  All threads of the CTA call;
 * every CTA of the grid raises the signal once, so the receiver expects gridDim.x per call --
 * launch with one CTA when a single increment per put is wanted. */
template <typename W>
__device__ __forceinline__ void devicePutSignal(const W& w, int peer, size_t peerOffset, const void* local,
                                                size_t bytes) {
  if (!UCCL_DEVICE_ACCESS_OK(w, 1, peer, peerOffset, bytes)) return;  /* no signal for data that was not written */
  uccl_device::copy_bytes(w.remotePtrs[peer] + peerOffset, static_cast<const char*>(local), bytes);
  __syncthreads();
  if (threadIdx.x == 0) uccl_device::signal_add(w.remoteSignals[peer] + w.myRank, 1ull);
}
/* Get, then bump the local counter of `peer` (completion marker for this rank's own waits). */
template <typename W>
__device__ __forceinline__ void deviceGetSignal(const W& w, int peer, size_t peerOffset, void* local, size_t bytes) {
  if (!UCCL_DEVICE_ACCESS_OK(w, 2, peer, peerOffset, bytes)) return;
  uccl_device::copy_bytes(static_cast<char*>(local), w.remotePtrs[peer] + peerOffset, bytes);
  __syncthreads();
  if (threadIdx.x == 0) uccl_device::signal_add(w.localSignals + peer, 1ull);
}
/* Wait until `peer` has signalled at least `expected` times in total.  Always bounded: returns
 * false when the window's time budget (ten seconds if the descriptor says 0) ran out.  Call from
 * one thread (or use the cooperative form). */
template <typename W>
__device__ __forceinline__ bool deviceWaitSignal(const W& w, int peer, unsigned long long expected) {
  const unsigned long long* p = w.localSignals + peer;
  if (uccl_device::signal_load(p) >= expected) return true;
  const unsigned long long budget = w.timeoutNs ? w.timeoutNs : uccl_device::kDefaultWaitNs;
  const unsigned long long t0 = uccl_device::globaltimer();
  unsigned int spins = 0;
  while (uccl_device::signal_load(p) < expected) {
    if ((++spins & 63u) == 0 && uccl_device::globaltimer() - t0 > budget) return false;
  }
  return true;
}
/* Thread 0 waits, the whole CTA learns the outcome. */
template <typename W>
__device__ __forceinline__ bool deviceWaitSignalCooperative(const W& w, int peer, unsigned long long expected) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = deviceWaitSignal(w, peer, expected) ? 1 : 0;
  __syncthreads();
  const bool r = ok != 0;
  __syncthreads();
  return r;
}
/* Wait for several peers at once; false as soon as one wait runs out. */
template <typename W>
__device__ __forceinline__ bool deviceWaitSignalMulti(const W& w, const int* peers, const unsigned long long* expected,
                                                      int n) {
  for (int i = 0; i < n; ++i)
    if (!deviceWaitSignal(w, peers[i], expected[i])) return false;
  return true;
}

/* ---- fused pull + reduce ------------------------------------------------------------------- */
/* result[i] = op(local[i], remote[i]) for `count` elements of T read at byte offset
 * `peerByteOffset` of `peer`'s window (rma_device.hpp:335-357).  The operands are widened to
 * fp32, combined, and rounded once; `result` may alias `local`.  Grid-stride: the whole grid
 * takes part. */
template <typename T, typename RedOp, typename W>
__device__ __forceinline__ void deviceGetReduce(const W& w, const T* local, T* result, size_t count, int peer,
                                                size_t peerByteOffset) {
  if (!UCCL_DEVICE_ACCESS_OK(w, 3, peer, peerByteOffset, count * sizeof(T))) return;
  const T* remote = reinterpret_cast<const T*>(w.remotePtrs[peer] + peerByteOffset);
  RedOp op;
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nth = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = tid; i < count; i += nth)
    result[i] = uccl_device::from_float<T>(op(uccl_device::to_float(local[i]), uccl_device::to_float(remote[i])));
}
/* local[i] += remote[i] for `count` floats. */
template <typename W>
__device__ __forceinline__ void deviceGetReduceF32(const W& w, int peer, size_t peerElemOffset, float* local,
                                                   size_t count) {
  deviceGetReduce<float, ucclDeviceSum>(w, local, local, count, peer, peerElemOffset * sizeof(float));
}

#ifdef UCCL_DEVICE_CHECKS
/* Host: copies the record of refused accesses (see the top of this file) into out[4] and clears it. */
static inline cudaError_t ucclDeviceCheckRead(unsigned long long out[4]) {
  cudaError_t e = cudaMemcpyFromSymbol(out, uccl_device::g_check_record, 4 * sizeof(unsigned long long));
  if (e != cudaSuccess) return e;
  const unsigned long long zero[4] = {0, 0, 0, 0};
  return cudaMemcpyToSymbol(uccl_device::g_check_record, zero, sizeof(zero));
}
#endif

#endif /* __CUDACC__ */
#endif /* UCCL_DEVICE_CUH_ */
