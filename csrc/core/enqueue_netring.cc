// Host launcher of the GPU-driven network ring all-reduce.
#include <string.h>

#include "../kernels/net_ring.h"
#include "enqueue.h"
#include "log.h"

namespace uccl {

ucclResult_t launchNetRingAllReduce(Comm* c, const CollOp& op) {
  const size_t es = dataTypeSize(op.dtype);
  if (op.send != op.recv &&
      cudaMemcpyAsync(op.recv, op.send, op.count * es, cudaMemcpyDeviceToDevice, op.stream) != cudaSuccess) {
    commSetError(c, "cudaMemcpyAsync failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  NetRingArgs a;
  memset(&a, 0, sizeof(a));
  a.dc = c->dev;
  a.buf = static_cast<char*>(op.recv);
  a.dtype = op.dtype == ucclFloat16 ? DEVDT_F16 : (op.dtype == ucclBfloat16 ? DEVDT_BF16 : DEVDT_F32);
  a.nranks = c->nRanks;
  a.ringPos = c->channels[0].index;
  a.prevRank = c->channels[0].prev;
  a.nextRank = c->channels[0].next;
  a.slotBytes = c->channels[0].send.slotBytes;
  int nch = 0;
  for (Channel& ch : c->channels)
    if (ch.netReady) ++nch;
  if (nch == 0) {
    commSetError(c, "network ring is not connected");
    return ucclInternalError;
  }
  // small messages do not need every channel
  const size_t perCh = (a.slotBytes / es) * static_cast<size_t>(c->nRanks);
  int use = static_cast<int>(std::min<size_t>(nch, (op.count + perCh - 1) / perCh));
  if (use < 1) use = 1;
  a.nChannels = use;
  size_t off = 0;
  for (int i = 0; i < use; ++i) {
    Channel& ch = c->channels[i];
    const size_t len = op.count / use + (static_cast<size_t>(i) < op.count % use ? 1 : 0);
    a.ch[i].sendFifo = ch.send.fifoDev;
    a.ch[i].recvFifo = ch.recv.fifoDev;
    a.ch[i].sendBounce = ch.send.bounceDev;
    a.ch[i].recvBounce = ch.recv.bounceDev;
    a.ch[i].elemOff = off;
    a.ch[i].elemCount = len;
    off += len;
  }
  cudaError_t e = launchNetRingKernel(a, op.stream);
  if (e != cudaSuccess) {
    commSetError(c, "net ring kernel launch failed: %s", cudaGetErrorString(e));
    return ucclSystemError;
  }
  return ucclSuccess;
}

}  // namespace uccl
