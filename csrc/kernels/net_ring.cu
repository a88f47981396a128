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

enum NetRecvMode : int { NET_RECV_NONE = 0, NET_RECV_COPY = 1, NET_RECV_SUM = 2 };

struct NetChan {
  NetSide snd, rcv;
  uint64_t rcvDone;  // receive steps consumed so far (same value in every thread)
  int prevRank, nextRank;
};

// One hop of the ring for one channel: sends `sendElems` elements from sendSrc (unless null) and
// receives `recvElems`: COPY -> recvDst = incoming, SUM -> recvDst += incoming.  Both directions
// move in pieces of one bounce slot and are interleaved piece by piece, with up to UCCL_STEPS
// receives posted ahead.  `recvFirst` handles piece j's receive before its send, for a rank that
// forwards what it has just received (sendSrc then points into recvDst).  The roles are the
// reference's sendViaBounce / postRecv / waitRecv / reduceFromBounceRecv / copyFromBounceRecv
// (src/device/primitives.hpp:223-341).  Returns false when a wait gave up (all threads agree).
template <int DT>
__device__ bool net_xfer(const DevComm& dc, NetChan& c, const char* sendSrc, size_t sendElems, int recvMode, char* recvDst,
                         size_t recvElems, bool recvFirst) {
  using V = Vec<DT>;
  __shared__ int s_ok;
  const size_t slotBytes = c.snd.slotBytes;
  const size_t slotElems = slotBytes / V::ES;
  const size_t nsubS = sendSrc ? (sendElems + slotElems - 1) / slotElems : 0;
  const size_t nsubR = recvMode != NET_RECV_NONE ? (recvElems + slotElems - 1) / slotElems : 0;
  const size_t nsub = max(nsubS, nsubR);
  // Receive steps of this hop occupy FIFO steps [recvBase, recvBase + nsubR); every thread knows
  // recvBase, only the leader's rcv.step follows the actual posting.
  const uint64_t recvBase = c.rcvDone;
  size_t recvPosted = 0;
  auto doSend = [&](size_t j) -> bool {
    const size_t e = min(slotElems, sendElems - j * slotElems);
    if (threadIdx.x == 0)
      s_ok = c.snd.step >= UCCL_STEPS ? net_wait_head(c.snd, c.snd.step - UCCL_STEPS + 1, dc, c.nextRank) : 1;
    __syncthreads();
    if (!s_ok) return false;
    char* slot = c.snd.bounce + (c.snd.step % UCCL_STEPS) * slotBytes;
    block_copy(slot, sendSrc + j * slotElems * V::ES, e * V::ES);
    __syncthreads();
    if (threadIdx.x == 0) net_post(c.snd, FIFO_SEND, e * V::ES);
    ++c.snd.step;
    return true;
  };
  auto doRecv = [&](size_t j) -> bool {
    const size_t e = min(slotElems, recvElems - j * slotElems);
    const uint64_t myStep = recvBase + j;
    __syncthreads();
    if (threadIdx.x == 0) s_ok = net_wait_head(c.rcv, myStep + 1, dc, c.prevRank);
    __syncthreads();
    if (!s_ok) return false;
    const char* slot = c.rcv.bounce + (myStep % UCCL_STEPS) * slotBytes;
    char* dst = recvDst + j * slotElems * V::ES;
    if (recvMode == NET_RECV_SUM) {
      for (size_t i = threadIdx.x; i < e; i += blockDim.x)
        V::store1(dst + i * V::ES, V::load1(dst + i * V::ES) + V::load1(slot + i * V::ES));
    } else {
      block_copy(dst, slot, e * V::ES);
    }
    __syncthreads();
    return true;
  };
  for (size_t j = 0; j < nsub; ++j) {
    // keep up to UCCL_STEPS receives posted ahead of consumption
    if (threadIdx.x == 0) {
      while (recvPosted < nsubR && recvPosted < j + UCCL_STEPS) {
        const size_t e = min(slotElems, recvElems - recvPosted * slotElems);
        net_post(c.rcv, FIFO_RECV, e * V::ES);
        ++c.rcv.step;
        ++recvPosted;
      }
    }
    if (recvFirst) {
      if (j < nsubR && !doRecv(j)) return false;
      if (j < nsubS && !doSend(j)) return false;
    } else {
      if (j < nsubS && !doSend(j)) return false;
      if (j < nsubR && !doRecv(j)) return false;
    }
  }
  c.rcvDone += nsubR;
  return true;
}

// The five collectives of the network ring as sequences of hops (see NetRingColl for what `buf`
// holds).  All-reduce follows the reference's schedule (src/algorithms/ring.cc:199-274): n - 1
// reduce-scatter hops, then n - 1 all-gather hops; all-gather and reduce-scatter are its two
// halves on whole rank chunks; broadcast and reduce are pipelines along the ring that start or
// end at the root.
template <int DT>
__device__ void net_ring_run(const NetRingArgs& a, const NetRingChannel& ch) {
  using V = Vec<DT>;
  const DevComm& dc = a.dc;
  const int n = a.nranks, r = a.ringPos;
  __shared__ uint64_t s_sendStep, s_recvStep;
  if (threadIdx.x == 0) {
    s_sendStep = ptx::ld_acquire_sys_u64(&ch.sendFifo->tail);
    s_recvStep = ptx::ld_acquire_sys_u64(&ch.recvFifo->tail);
  }
  __syncthreads();
  NetChan c;
  c.snd = NetSide{ch.sendFifo, ch.sendBounce, a.slotBytes, s_sendStep};
  c.rcv = NetSide{ch.recvFifo, ch.recvBounce, a.slotBytes, s_recvStep};
  c.rcvDone = s_recvStep;
  c.prevRank = a.prevRank;
  c.nextRank = a.nextRank;
  auto pos = [&](int p) { return ((p % n) + n) % n; };
  bool ok = true;
  if (a.coll == NET_RING_ALLREDUCE) {
    char* buf = a.buf + ch.elemOff * V::ES;
    auto chunk = [&](int p, char** base, size_t* len) {
      size_t o, l;
      split(ch.elemCount, n, pos(p), &o, &l);
      *base = buf + o * V::ES;
      *len = l;
    };
    for (int phase = 0; phase < 2 && ok; ++phase)
      for (int s = 0; s < n - 1 && ok; ++s) {
        char *sb, *rb;
        size_t sl, rl;
        chunk(phase == 0 ? r - s : r + 1 - s, &sb, &sl);
        chunk(phase == 0 ? r - s - 1 : r - s, &rb, &rl);
        ok = net_xfer<DT>(dc, c, sb, sl, phase == 0 ? NET_RECV_SUM : NET_RECV_COPY, rb, rl, false);
      }
  } else if (a.coll == NET_RING_ALLGATHER || a.coll == NET_RING_REDUCESCATTER) {
    // the chunk at ring position p belongs to rank ringRanks[p]; this channel moves its slice of it
    auto chunk = [&](int p) { return a.buf + (static_cast<size_t>(a.ringRanks[pos(p)]) * a.chunkElems + ch.elemOff) * V::ES; };
    const bool gather = a.coll == NET_RING_ALLGATHER;
    for (int s = 0; s < n - 1 && ok; ++s)
      ok = net_xfer<DT>(dc, c, chunk(gather ? r - s : r - 1 - s), ch.elemCount, gather ? NET_RECV_COPY : NET_RECV_SUM,
                        chunk(gather ? r - s - 1 : r - 2 - s), ch.elemCount, false);
  } else {
    char* buf = a.buf + ch.elemOff * V::ES;
    const int d = pos(r - a.rootPos);  // distance from the root along the ring
    if (a.coll == NET_RING_BROADCAST) {
      if (d == 0) ok = net_xfer<DT>(dc, c, buf, ch.elemCount, NET_RECV_NONE, nullptr, 0, false);
      else ok = net_xfer<DT>(dc, c, d == n - 1 ? nullptr : buf, ch.elemCount, NET_RECV_COPY, buf, ch.elemCount, true);
    } else {
      // reduce: the rank after the root starts the chain, every rank adds its part, the root ends it
      if (d == 1) ok = net_xfer<DT>(dc, c, buf, ch.elemCount, NET_RECV_NONE, nullptr, 0, false);
      else ok = net_xfer<DT>(dc, c, d == 0 ? nullptr : buf, ch.elemCount, NET_RECV_SUM, buf, ch.elemCount, true);
    }
  }
  // all sends must have left the bounce slots before the kernel ends (the next producer may be
  // the host, which reuses them)
  if (ok && threadIdx.x == 0 && c.snd.step > 0) net_wait_head(c.snd, c.snd.step, dc, a.nextRank);
}

template <int DT>
__global__ void __launch_bounds__(kThreads, 1) net_ring_kernel(const __grid_constant__ NetRingArgs a) {
  if (static_cast<int>(blockIdx.x) >= a.nChannels) return;
  if (a.nranks < 2 || a.ch[blockIdx.x].elemCount == 0) return;
  net_ring_run<DT>(a, a.ch[blockIdx.x]);
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
