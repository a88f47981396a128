// Collectives of a GPU communicator whose ranks cannot reach each other over NVLink (several
// hosts, UCCL_FORCE_NET=1, or no peer access): the data crosses the network plugin.
//
// All-reduce, all-gather, reduce-scatter, broadcast and reduce run as a persistent ring kernel
// that talks to the proxy thread through mapped FIFOs (kernels/net_ring.cu), the arrangement of
// the reference's net ring (src/algorithms/ring.cc:170-279), stream-ordered.  All-to-all and
// point-to-point batches, which need connections beyond the ring neighbours and which the
// reference does not offer over the network at all, are staged through pinned host memory and
// handed to the host transfer loop; those two wait for the stream.
#include <string.h>

#include "../host/host_coll.h"
#include "enqueue.h"
#include "log.h"

namespace uccl {

// the ring kernel and its launcher (enqueue_netring.cc)
bool netRingHandles(const CollOp& op);
ucclResult_t launchNetRing(Comm* c, const CollOp& op);

namespace {

struct Pinned {
  void* p = nullptr;
  explicit Pinned(size_t n) {
    if (n && cudaMallocHost(&p, n) != cudaSuccess) {
      (void)cudaGetLastError();
      p = nullptr;
    }
  }
  ~Pinned() { if (p) cudaFreeHost(p); }
};

ucclResult_t cudaFail(Comm* c, const char* what) {
  commSetError(c, "%s: %s", what, cudaGetErrorString(cudaGetLastError()));
  return ucclSystemError;
}

}  // namespace

ucclResult_t enqueueNetGpu(Comm* c, const CollOp& op) {
  const size_t es = dataTypeSize(op.dtype);
  const int n = c->nRanks;
  if (netRingHandles(op) && getenv("UCCL_NET_STAGED") == nullptr) return launchNetRing(c, op);

  size_t sendBytes = op.count * es, recvBytes = op.count * es;
  if (op.kind == ucclCollAllGather) recvBytes *= n;
  if (op.kind == ucclCollReduceScatter) sendBytes *= n;
  if (op.kind == ucclCollAllToAll) { sendBytes *= n; recvBytes *= n; }
  Pinned hs(sendBytes), hr(recvBytes);
  if (!hs.p || !hr.p) return cudaFail(c, "pinned staging allocation failed");
  const bool needSend = !(op.kind == ucclCollBroadcast && c->rank != op.root);
  if (needSend && cudaMemcpyAsync(hs.p, op.send, sendBytes, cudaMemcpyDeviceToHost, op.stream) != cudaSuccess)
    return cudaFail(c, "device-to-host staging copy failed");
  if (cudaStreamSynchronize(op.stream) != cudaSuccess) return cudaFail(c, "stream synchronisation failed");
  CollOp h = op;
  h.send = hs.p;
  h.recv = hr.p;
  ucclResult_t r;
  switch (op.kind) {
    case ucclCollAllReduce: r = hostAllReduce(c, h.send, h.recv, op.count, op.dtype); break;
    case ucclCollAllGather: r = hostAllGather(c, h.send, h.recv, op.count, op.dtype); break;
    case ucclCollReduceScatter: r = hostReduceScatter(c, h.send, h.recv, op.count, op.dtype); break;
    case ucclCollBroadcast: r = hostBroadcast(c, h.send, h.recv, op.count, op.dtype, op.root); break;
    case ucclCollReduce: r = hostReduce(c, h.send, h.recv, op.count, op.dtype, op.root); break;
    case ucclCollAllToAll: r = hostAllToAll(c, h.send, h.recv, op.count, op.dtype); break;
    default: return ucclInternalError;
  }
  if (r != ucclSuccess) return r;
  const bool haveResult = !(op.kind == ucclCollReduce && c->rank != op.root);
  if (haveResult) {
    if (cudaMemcpyAsync(op.recv, hr.p, recvBytes, cudaMemcpyHostToDevice, op.stream) != cudaSuccess)
      return cudaFail(c, "host-to-device staging copy failed");
    if (cudaStreamSynchronize(op.stream) != cudaSuccess) return cudaFail(c, "stream synchronisation failed");
  }
  return ucclSuccess;
}

ucclResult_t enqueueNetGpuP2p(Comm* c, const std::vector<CollOp>& ops) {
  std::vector<std::unique_ptr<Pinned>> bufs;
  std::vector<HostP2pOp> hops;
  cudaStream_t stream = ops[0].stream;
  for (const CollOp& op : ops) {
    const size_t bytes = op.count * dataTypeSize(op.dtype);
    bufs.emplace_back(new Pinned(bytes));
    if (!bufs.back()->p) return cudaFail(c, "pinned staging allocation failed");
    if (op.isSend && cudaMemcpyAsync(bufs.back()->p, op.send, bytes, cudaMemcpyDeviceToHost, stream) != cudaSuccess)
      return cudaFail(c, "device-to-host staging copy failed");
    hops.push_back({op.isSend, op.root, bufs.back()->p, bufs.back()->p, bytes});
  }
  if (cudaStreamSynchronize(stream) != cudaSuccess) return cudaFail(c, "stream synchronisation failed");
  ucclResult_t r = hostSendRecv(c, hops);
  if (r != ucclSuccess) return r;
  for (size_t i = 0; i < ops.size(); ++i) {
    if (ops[i].isSend) continue;
    if (cudaMemcpyAsync(ops[i].recv, bufs[i]->p, hops[i].bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess)
      return cudaFail(c, "host-to-device staging copy failed");
  }
  if (cudaStreamSynchronize(stream) != cudaSuccess) return cudaFail(c, "stream synchronisation failed");
  return ucclSuccess;
}

}  // namespace uccl
