// Work queue between a producer that cannot make system calls (a persistent GPU kernel, or the
// CPU-rank ring loop) and the proxy thread that drives the network plugin.
//
// The reference's queue (src/include/fifo.h:19-47) keeps a per-entry `done` flag and a
// `request` pointer inside the shared structure and marks fields `volatile`.  Here the shared
// part holds only two monotonically increasing 64-bit counters and the entry payloads:
//   tail  written by the producer : number of operations posted so far
//   head  written by the proxy    : number of operations completed so far (in order)
// Entry i lives in slot i % UCCL_STEPS; the producer may post while tail - head < UCCL_STEPS.
// All proxy-private state (plugin request handles, "already posted" count) stays outside the
// shared memory, so an operation that completes inside isend/irecv cannot be mistaken for one
// that was never posted.  Both counters are accessed with acquire/release atomics on the host
// and ld.acquire.sys / st.release.sys on the device; the structure lives in mapped pinned host
// memory when the producer is a kernel.
#pragma once
#include <stdint.h>

#include "uccl.h"

namespace uccl {

enum FifoOp : uint32_t { FIFO_SEND = 0, FIFO_RECV = 1, FIFO_PUT = 2, FIFO_SIGNAL = 3, FIFO_WAIT = 4 };

struct FifoEntry {
  uint32_t op;      // FifoOp
  uint32_t slot;    // bounce slot index the payload sits in / lands in
  uint64_t bytes;   // payload size (0 for SIGNAL)
  uint64_t step;    // producer's step number, echoed in traces
  uint64_t result;  // written by the proxy before head advances: bytes actually moved
};

struct alignas(64) ConnFifo {
  alignas(64) uint64_t tail;  // producer
  alignas(64) uint64_t head;  // proxy
  alignas(64) uint64_t error; // proxy: non-zero ucclResult_t once the connection failed
  alignas(64) FifoEntry entries[UCCL_STEPS];
};

// Host-side accessors (the device side uses ld.acquire.sys / st.release.sys, kernels/net_ring.cu).
inline uint64_t fifoLoadAcquire(const uint64_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline void fifoStoreRelease(uint64_t* p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }

}  // namespace uccl
