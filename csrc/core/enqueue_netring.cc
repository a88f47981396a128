// Host launcher of the GPU-driven network ring: all-reduce, all-gather, reduce-scatter, broadcast
// and reduce run as one persistent kernel that talks to the proxy thread through mapped FIFOs
// (kernels/net_ring.cu), stream-ordered from end to end.  The reference's network kernel offers
// all-reduce only (src/algorithms/ring.cc:170-279; enqueue.cc:431,544 has no network variant of
// the other two).
#include <string.h>

#include <algorithm>

#include "../kernels/net_ring.h"
#include "enqueue.h"
#include "log.h"

namespace uccl {

namespace {

ucclResult_t cudaFail(Comm* c, const char* what) {
  commSetError(c, "%s: %s", what, cudaGetErrorString(cudaGetLastError()));
  return ucclSystemError;
}

// Device scratch that outlives the call (the kernel works on it after the launcher returned).
// Growing it is the only moment the stream is waited for.
ucclResult_t netScratch(Comm* c, size_t bytes, cudaStream_t s, char** out) {
  if (c->netScratchBytes < bytes) {
    if (c->netScratch) {
      if (cudaStreamSynchronize(s) != cudaSuccess) return cudaFail(c, "stream synchronisation failed");
      cudaFree(c->netScratch);
      c->netScratch = nullptr;
      c->netScratchBytes = 0;
    }
    const size_t want = std::max<size_t>(bytes, 1u << 20);
    if (cudaMalloc(&c->netScratch, want) != cudaSuccess) return cudaFail(c, "network ring scratch allocation failed");
    c->netScratchBytes = want;
  }
  *out = static_cast<char*>(c->netScratch);
  return ucclSuccess;
}

ucclResult_t copyAsync(Comm* c, void* dst, const void* src, size_t bytes, cudaStream_t s) {
  if (bytes == 0 || dst == src) return ucclSuccess;
  if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s) != cudaSuccess) return cudaFail(c, "cudaMemcpyAsync failed");
  return ucclSuccess;
}

}  // namespace

// True when the ring kernel can carry this operation (everything but all-to-all and
// point-to-point; copy-only collectives need a byte count that is a multiple of two).
bool netRingHandles(const CollOp& op) {
  switch (op.kind) {
    case ucclCollAllReduce:
    case ucclCollReduceScatter:
    case ucclCollReduce: return true;
    case ucclCollAllGather:
    case ucclCollBroadcast: {
      const size_t es = dataTypeSize(op.dtype);
      return es >= 2 || (op.count % 2) == 0;
    }
    default: return false;
  }
}

ucclResult_t launchNetRing(Comm* c, const CollOp& op) {
  const int n = c->nRanks;
  size_t es = dataTypeSize(op.dtype);
  size_t count = op.count;
  int dtype = op.dtype == ucclFloat16 ? DEVDT_F16 : (op.dtype == ucclBfloat16 ? DEVDT_BF16 : DEVDT_F32);
  if (op.dtype != ucclFloat16 && op.dtype != ucclBfloat16 && op.dtype != ucclFloat32) {
    // copy-only element types travel as 4- or 2-byte words
    const size_t bytes = count * es;
    es = (bytes % 4 == 0) ? 4 : 2;
    count = bytes / es;
    dtype = es == 4 ? DEVDT_F32 : DEVDT_F16;
  }
  cudaStream_t s = op.stream;
  const Channel& ch0 = c->channels[0];
  NetRingArgs a;
  memset(&a, 0, sizeof(a));
  a.dc = c->dev;
  a.dtype = dtype;
  a.nranks = n;
  a.ringPos = ch0.index;
  a.prevRank = ch0.prev;
  a.nextRank = ch0.next;
  a.slotBytes = ch0.send.slotBytes;
  for (int p = 0; p < n; ++p) a.ringRanks[p] = ch0.userRanks[((p - ch0.index) % n + n) % n];
  ucclResult_t r;
  size_t sliceElems = count;  // what is cut over the channels
  char* scratch = nullptr;
  switch (op.kind) {
    case ucclCollAllReduce:
      a.coll = NET_RING_ALLREDUCE;
      if ((r = copyAsync(c, op.recv, op.send, count * es, s)) != ucclSuccess) return r;
      a.buf = static_cast<char*>(op.recv);
      break;
    case ucclCollAllGather:
      a.coll = NET_RING_ALLGATHER;
      a.chunkElems = count;
      if ((r = copyAsync(c, static_cast<char*>(op.recv) + static_cast<size_t>(c->rank) * count * es, op.send, count * es, s)) != ucclSuccess)
        return r;
      a.buf = static_cast<char*>(op.recv);
      break;
    case ucclCollReduceScatter:
      // partial sums are built in a work copy of the input; my chunk is copied out afterwards
      a.coll = NET_RING_REDUCESCATTER;
      a.chunkElems = count;
      if ((r = netScratch(c, count * es * n, s, &scratch)) != ucclSuccess) return r;
      if ((r = copyAsync(c, scratch, op.send, count * es * n, s)) != ucclSuccess) return r;
      a.buf = scratch;
      break;
    case ucclCollBroadcast:
      a.coll = NET_RING_BROADCAST;
      if (c->rank == op.root && (r = copyAsync(c, op.recv, op.send, count * es, s)) != ucclSuccess) return r;
      a.buf = static_cast<char*>(op.recv);
      break;
    case ucclCollReduce:
      // every rank but the root adds into a work copy; the root adds into its receive buffer
      a.coll = NET_RING_REDUCE;
      if (c->rank == op.root) {
        if ((r = copyAsync(c, op.recv, op.send, count * es, s)) != ucclSuccess) return r;
        a.buf = static_cast<char*>(op.recv);
      } else {
        if ((r = netScratch(c, count * es, s, &scratch)) != ucclSuccess) return r;
        if ((r = copyAsync(c, scratch, op.send, count * es, s)) != ucclSuccess) return r;
        a.buf = scratch;
      }
      break;
    default: return ucclInternalError;
  }
  if (op.kind == ucclCollBroadcast || op.kind == ucclCollReduce) {
    a.rootPos = 0;
    for (int p = 0; p < n; ++p)
      if (a.ringRanks[p] == op.root) a.rootPos = p;
  }
  int nch = 0;
  for (Channel& ch : c->channels)
    if (ch.netReady) ++nch;
  if (nch == 0) {
    commSetError(c, "network ring is not connected");
    return ucclInternalError;
  }
  // small messages do not need every channel: at least one slot of work per hop and channel
  const size_t slotElems = std::max<size_t>(1, a.slotBytes / es);
  const size_t perCh = op.kind == ucclCollAllReduce ? slotElems * static_cast<size_t>(n) : slotElems;
  int use = static_cast<int>(std::min<size_t>(nch, (sliceElems + perCh - 1) / perCh));
  if (use < 1) use = 1;
  a.nChannels = use;
  size_t off = 0;
  for (int i = 0; i < use; ++i) {
    Channel& ch = c->channels[i];
    const size_t len = sliceElems / use + (static_cast<size_t>(i) < sliceElems % use ? 1 : 0);
    a.ch[i].sendFifo = ch.send.fifoDev;
    a.ch[i].recvFifo = ch.recv.fifoDev;
    a.ch[i].sendBounce = ch.send.bounceDev;
    a.ch[i].recvBounce = ch.recv.bounceDev;
    a.ch[i].elemOff = off;
    a.ch[i].elemCount = len;
    off += len;
  }
  cudaError_t e = launchNetRingKernel(a, s);
  if (e != cudaSuccess) {
    commSetError(c, "net ring kernel launch failed: %s", cudaGetErrorString(e));
    return ucclSystemError;
  }
  if (op.kind == ucclCollReduceScatter)
    return copyAsync(c, op.recv, scratch + static_cast<size_t>(c->rank) * count * es, count * es, s);
  return ucclSuccess;
}

}  // namespace uccl
