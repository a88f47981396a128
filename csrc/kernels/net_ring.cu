// Ring all-reduce across the network plugin, driven from the GPU: a persistent kernel (one CTA
// per channel) fills bounce slots, posts send / receive descriptors into FIFOs that live in mapped
// pinned host memory, and consumes completions published by the proxy thread.
//
// Same roles as the reference's net kernel and its NetPrimitives (src/algorithms/ring.cc:170-279,
// src/device/primitives.hpp:190-361: sendViaBounce / postRecv / waitRecv / reduceFromBounceRecv /
// copyFromBounceRecv), with two changes: completion is read from the FIFO's monotonic head counter
// instead of per-entry done flags, and every wait (slot free, receive complete) has a deadline and
// watches the connection's error word and the abort word, where the reference spins without
// bound (primitives.hpp:230,274,305).
#include "../transport/fifo.h"
#include "coll_device.cuh"
#include "net_ring.h"

namespace uccl {
namespace dev {

struct NetSide {
  ConnFifo* fifo;
  char* bounce;
  size_t slotBytes;
  uint64_t step;  // next step to post (== fifo->tail when this CTA is the only producer)
};

__device__ __forceinline__ bool net_wait_head(NetSide& s, uint64_t need, const DevComm& dc, int peer) {
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (ptx::ld_acquire_sys_u64(&s.fifo->head) < need) {
    if ((++spins & 15u) == 0) {
      if (ptx::ld_relaxed_sys_u64(&s.fifo->error) != 0 || aborted(dc)) return false;
      if (ptx::globaltimer_ns() - t0 > dc.timeoutNs) {
        record_status(dc, DEV_TIMEOUT_NET, peer, static_cast<uint32_t>(need));
        return false;
      }
    }
    __nanosleep(200);
  }
  return true;
}

// leader thread: publish the descriptor of the next step
__device__ __forceinline__ void net_post(NetSide& s, uint32_t op, size_t bytes) {
  FifoEntry* e = &s.fifo->entries[s.step % UCCL_STEPS];
  e->op = op;
  e->slot = static_cast<uint32_t>(s.step % UCCL_STEPS);
  e->bytes = bytes;
  e->step = s.step;
  e->result = 0;
  ptx::fence_sys();
  ptx::st_release_sys_u64(&s.fifo->tail, s.step + 1);
}

template <int DT>
__device__ void net_ring_allreduce(const NetRingArgs& a, const NetRingChannel& ch) {
  using V = Vec<DT>;
  const DevComm& dc = a.dc;
  const int n = a.nranks, r = a.ringPos;
  __shared__ int s_ok;
  __shared__ uint64_t s_sendStep, s_recvStep;
  if (threadIdx.x == 0) {
    s_sendStep = ptx::ld_acquire_sys_u64(&ch.sendFifo->tail);
    s_recvStep = ptx::ld_acquire_sys_u64(&ch.recvFifo->tail);
  }
  __syncthreads();
  NetSide snd{ch.sendFifo, ch.sendBounce, a.slotBytes, s_sendStep};
  NetSide rcv{ch.recvFifo, ch.recvBounce, a.slotBytes, s_recvStep};
  char* buf = a.buf + ch.elemOff * V::ES;
  const size_t count = ch.elemCount;
  const size_t slotElems = a.slotBytes / V::ES;
  uint64_t rcvDone = s_recvStep;  // receive steps posted before this ring step (same in all threads)

  for (int phase = 0; phase < 2; ++phase) {
    for (int s = 0; s < n - 1; ++s) {
      const int sc = phase == 0 ? ((r - s) % n + n) % n : ((r + 1 - s) % n + n) % n;
      const int rc = phase == 0 ? ((r - s - 1) % n + n) % n : ((r - s) % n + n) % n;
      size_t so, sl, ro, rl;
      split(count, n, sc, &so, &sl);
      split(count, n, rc, &ro, &rl);
      const size_t nsubS = (sl + slotElems - 1) / slotElems, nsubR = (rl + slotElems - 1) / slotElems;
      const size_t nsub = max(nsubS, nsubR);
      // Receive steps of this ring step occupy FIFO steps [recvBase, recvBase + nsubR); every
      // thread knows recvBase, only the leader's rcv.step follows the actual posting.
      const uint64_t recvBase = rcvDone;
      size_t recvPosted = 0;
      for (size_t j = 0; j < nsub; ++j) {
        // keep up to UCCL_STEPS receives posted ahead of consumption
        if (threadIdx.x == 0) {
          while (recvPosted < nsubR && recvPosted < j + UCCL_STEPS) {
            const size_t e = min(slotElems, rl - recvPosted * slotElems);
            net_post(rcv, FIFO_RECV, e * V::ES);
            ++rcv.step;
            ++recvPosted;
          }
        }
        if (j < nsubS) {
          const size_t e = min(slotElems, sl - j * slotElems);
          if (threadIdx.x == 0)
            s_ok = snd.step >= UCCL_STEPS ? net_wait_head(snd, snd.step - UCCL_STEPS + 1, dc, a.nextRank) : 1;
          __syncthreads();
          if (!s_ok) return;
          char* slot = snd.bounce + (snd.step % UCCL_STEPS) * a.slotBytes;
          const char* src = buf + (so + j * slotElems) * V::ES;
          block_copy(slot, src, e * V::ES);
          __syncthreads();
          if (threadIdx.x == 0) net_post(snd, FIFO_SEND, e * V::ES);
          ++snd.step;
        }
        if (j < nsubR) {
          const size_t e = min(slotElems, rl - j * slotElems);
          const uint64_t myStep = recvBase + j;
          __syncthreads();
          if (threadIdx.x == 0) s_ok = net_wait_head(rcv, myStep + 1, dc, a.prevRank);
          __syncthreads();
          if (!s_ok) return;
          const char* slot = rcv.bounce + (myStep % UCCL_STEPS) * a.slotBytes;
          char* dst = buf + (ro + j * slotElems) * V::ES;
          if (phase == 0) {
            for (size_t i = threadIdx.x; i < e; i += blockDim.x)
              V::store1(dst + i * V::ES, V::load1(dst + i * V::ES) + V::load1(slot + i * V::ES));
          } else {
            block_copy(dst, slot, e * V::ES);
          }
          __syncthreads();
        }
      }
      rcvDone += nsubR;
    }
  }
  // all sends must have left the bounce slots before the kernel ends (the next producer may be
  // the host, which reuses them)
  if (threadIdx.x == 0 && snd.step > 0) net_wait_head(snd, snd.step, dc, a.nextRank);
}

template <int DT>
__global__ void __launch_bounds__(kThreads, 1) net_ring_kernel(const __grid_constant__ NetRingArgs a) {
  if (static_cast<int>(blockIdx.x) >= a.nChannels) return;
  net_ring_allreduce<DT>(a, a.ch[blockIdx.x]);
}

}  // namespace dev

cudaError_t launchNetRingKernel(const NetRingArgs& a, cudaStream_t stream) {
  switch (a.dtype) {
    case DEVDT_F16: dev::net_ring_kernel<dev::DT_F16><<<a.nChannels, dev::kThreads, 0, stream>>>(a); break;
    case DEVDT_BF16: dev::net_ring_kernel<dev::DT_BF16><<<a.nChannels, dev::kThreads, 0, stream>>>(a); break;
    case DEVDT_F32: dev::net_ring_kernel<dev::DT_F32><<<a.nChannels, dev::kThreads, 0, stream>>>(a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace uccl
