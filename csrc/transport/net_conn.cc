#include "net_conn.h"

#include <sched.h>
#include <stdlib.h>
#include <string.h>

#include "../core/comm.h"
#include "../core/log.h"

namespace uccl {

namespace {
constexpr int kMeshTag = 7000;

uint64_t makeTag(int src, int dst, int channel) {
  return (static_cast<uint64_t>(channel + 1) << 56) | (static_cast<uint64_t>(src) << 28) | static_cast<uint64_t>(dst);
}

void* hostAlloc(Comm* comm, size_t bytes, void** devAlias) {
  void* p = nullptr;
  if (comm->backend == BACKEND_CUDA) {
    if (cudaHostAlloc(&p, bytes, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    void* d = nullptr;
    if (cudaHostGetDevicePointer(&d, p, 0) != cudaSuccess) {
      (void)cudaGetLastError();
      cudaFreeHost(p);
      return nullptr;
    }
    *devAlias = d;
  } else {
    if (posix_memalign(&p, 4096, bytes) != 0) return nullptr;
    *devAlias = p;
  }
  memset(p, 0, bytes);
  return p;
}

void hostFree(Comm* comm, void* p) {
  if (!p) return;
  if (comm->backend == BACKEND_CUDA) cudaFreeHost(p);
  else free(p);
}

void registerConn(Comm* comm, NetConn* c) {
  std::lock_guard<std::mutex> lk(comm->netMu);
  comm->allConns.push_back(c);
}

ucclResult_t regSlots(Comm* comm, NetConn* c) {
  for (int s = 0; s < UCCL_STEPS; ++s) {
    ucclResult_t r = comm->net->regMr(c->netComm, c->bounce + s * c->slotBytes, c->slotBytes, UCCL_PTR_HOST,
                                      &c->mhandle[s]);
    if (r != ucclSuccess) {
      commSetError(comm, "plugin %s refused to register a bounce slot", comm->net->name);
      return r;
    }
  }
  return ucclSuccess;
}

ucclResult_t acceptLoop(Comm* comm, NetConn* c) {
  const uint64_t dl = nowMs() + comm->cfg.bootstrapTimeoutMs;
  while (true) {
    ucclResult_t r = comm->net->accept(c->listenComm, &c->netComm);
    if (r == ucclSuccess) break;
    if (r != ucclInProgress) return r;
    if (nowMs() > dl || comm->abortFlag.load()) {
      commSetError(comm, "rank %d never connected its network channel", c->peer);
      return ucclRemoteError;
    }
    comm->net->progress(comm->netContext);
    sched_yield();
  }
  comm->net->closeListen(c->listenComm);
  c->listenComm = nullptr;
  return ucclSuccess;
}
}  // namespace

ucclResult_t netConnAlloc(Comm* comm, NetConn* c, bool isSend, int peer, int channel) {
  c->isSend = isSend;
  c->peer = peer;
  c->channel = channel;
  c->slotBytes = comm->cfg.netChunkBytes;
  void* dev = nullptr;
  c->fifo = static_cast<ConnFifo*>(hostAlloc(comm, sizeof(ConnFifo), &dev));
  c->fifoDev = static_cast<ConnFifo*>(dev);
  c->bounce = static_cast<char*>(hostAlloc(comm, c->slotBytes * UCCL_STEPS, &dev));
  c->bounceDev = static_cast<char*>(dev);
  if (!c->fifo || !c->bounce) {
    commSetError(comm, "out of pinned host memory for network buffers");
    return ucclSystemError;
  }
  return ucclSuccess;
}

void netConnFree(Comm* comm, NetConn* c) {
  if (comm->net && c->netComm) {
    for (int s = 0; s < UCCL_STEPS; ++s)
      if (c->mhandle[s]) comm->net->deregMr(c->netComm, c->mhandle[s]);
    if (c->isSend) comm->net->closeSend(c->netComm);
    else comm->net->closeRecv(c->netComm);
  }
  if (comm->net && c->listenComm) comm->net->closeListen(c->listenComm);
  hostFree(comm, c->fifo);
  hostFree(comm, c->bounce);
  *c = NetConn();
}

ucclResult_t netSetupRings(Comm* comm) {
  const int n = comm->nRanks, nch = comm->nChannels;
  if (!comm->net || n <= 1) return ucclSuccess;
  std::vector<char> handles(static_cast<size_t>(n) * nch * UCCL_NET_HANDLE_BYTES, 0);
  ucclResult_t r;
  for (int ch = 0; ch < nch; ++ch) {
    Channel& c = comm->channels[ch];
    if ((r = netConnAlloc(comm, &c.recv, false, c.prev, ch)) != ucclSuccess) return r;
    if ((r = netConnAlloc(comm, &c.send, true, c.next, ch)) != ucclSuccess) return r;
    char* mine = handles.data() + (static_cast<size_t>(comm->rank) * nch + ch) * UCCL_NET_HANDLE_BYTES;
    if ((r = comm->net->listen(comm->netContext, mine, &c.recv.listenComm)) != ucclSuccess) {
      commSetError(comm, "plugin %s: listen failed", comm->net->name);
      return r;
    }
  }
  if ((r = comm->bootstrap.allGather(handles.data(), static_cast<size_t>(nch) * UCCL_NET_HANDLE_BYTES)) != ucclSuccess)
    return r;
  for (int ch = 0; ch < nch; ++ch) {
    Channel& c = comm->channels[ch];
    char* theirs = handles.data() + (static_cast<size_t>(c.next) * nch + ch) * UCCL_NET_HANDLE_BYTES;
    if ((r = comm->net->connect(comm->netContext, theirs, &c.send.netComm)) != ucclSuccess) {
      commSetError(comm, "plugin %s: connect to rank %d failed", comm->net->name, c.next);
      return r;
    }
  }
  for (int ch = 0; ch < nch; ++ch) {
    Channel& c = comm->channels[ch];
    if ((r = acceptLoop(comm, &c.recv)) != ucclSuccess) return r;
    comm->net->setTag(c.send.netComm, makeTag(comm->rank, c.next, ch));
    comm->net->setTag(c.recv.netComm, makeTag(c.prev, comm->rank, ch));
    if ((r = regSlots(comm, &c.send)) != ucclSuccess) return r;
    if ((r = regSlots(comm, &c.recv)) != ucclSuccess) return r;
    registerConn(comm, &c.send);
    registerConn(comm, &c.recv);
    c.netReady = true;
  }
  return comm->bootstrap.barrier();
}

// Both directions to `peers` at once.  Every rank named here must make the matching call.
ucclResult_t netEnsurePeers(Comm* comm, const std::vector<int>& peers) {
  if (!comm->net) return ucclInvalidUsage;
  if (comm->meshSend.empty()) {
    comm->meshSend.resize(comm->nRanks);
    comm->meshRecv.resize(comm->nRanks);
  }
  std::vector<int> todo;
  for (int p : peers)
    if (p != comm->rank && !comm->meshSend[p]) todo.push_back(p);
  if (todo.empty()) return ucclSuccess;
  ucclResult_t r;
  constexpr int kMeshChannel = 100;
  // 1. listen for each peer and tell it where
  for (int p : todo) {
    comm->meshRecv[p].reset(new NetConn());
    comm->meshSend[p].reset(new NetConn());
    if ((r = netConnAlloc(comm, comm->meshRecv[p].get(), false, p, kMeshChannel)) != ucclSuccess) return r;
    if ((r = netConnAlloc(comm, comm->meshSend[p].get(), true, p, kMeshChannel)) != ucclSuccess) return r;
    char handle[UCCL_NET_HANDLE_BYTES] = {0};
    if ((r = comm->net->listen(comm->netContext, handle, &comm->meshRecv[p]->listenComm)) != ucclSuccess) return r;
    if ((r = comm->bootstrap.send(p, kMeshTag, handle, sizeof(handle))) != ucclSuccess) return r;
  }
  // 2. connect to each peer's listener
  for (int p : todo) {
    char handle[UCCL_NET_HANDLE_BYTES];
    if ((r = comm->bootstrap.recv(p, kMeshTag, handle, sizeof(handle))) != ucclSuccess) return r;
    if ((r = comm->net->connect(comm->netContext, handle, &comm->meshSend[p]->netComm)) != ucclSuccess) {
      commSetError(comm, "plugin %s: connect to rank %d failed", comm->net->name, p);
      return r;
    }
  }
  // 3. accept
  for (int p : todo) {
    NetConn* rc = comm->meshRecv[p].get();
    NetConn* sc = comm->meshSend[p].get();
    if ((r = acceptLoop(comm, rc)) != ucclSuccess) return r;
    comm->net->setTag(sc->netComm, makeTag(comm->rank, p, kMeshChannel));
    comm->net->setTag(rc->netComm, makeTag(p, comm->rank, kMeshChannel));
    if ((r = regSlots(comm, sc)) != ucclSuccess) return r;
    if ((r = regSlots(comm, rc)) != ucclSuccess) return r;
    registerConn(comm, sc);
    registerConn(comm, rc);
  }
  return ucclSuccess;
}

ucclResult_t netGetSendConn(Comm* comm, int peer, NetConn** out) {
  ucclResult_t r = netEnsurePeers(comm, {peer});
  if (r != ucclSuccess) return r;
  *out = comm->meshSend[peer].get();
  return ucclSuccess;
}
ucclResult_t netGetRecvConn(Comm* comm, int peer, NetConn** out) {
  ucclResult_t r = netEnsurePeers(comm, {peer});
  if (r != ucclSuccess) return r;
  *out = comm->meshRecv[peer].get();
  return ucclSuccess;
}

void netTeardown(Comm* comm) {
  {
    std::lock_guard<std::mutex> lk(comm->netMu);
    comm->allConns.clear();
  }
  for (Channel& c : comm->channels) {
    netConnFree(comm, &c.send);
    netConnFree(comm, &c.recv);
    c.netReady = false;
  }
  for (auto& p : comm->meshSend)
    if (p) netConnFree(comm, p.get());
  for (auto& p : comm->meshRecv)
    if (p) netConnFree(comm, p.get());
  comm->meshSend.clear();
  comm->meshRecv.clear();
}

// ------------------------------------------------------------------ host-side producer
static ucclResult_t hostSpin(Comm* comm, NetConn* c, uint64_t needHead) {
  const uint64_t dl = nowMs() + comm->cfg.waitTimeoutMs;
  uint32_t spins = 0;
  while (fifoLoadAcquire(&c->fifo->head) < needHead) {
    const uint64_t err = __atomic_load_n(&c->fifo->error, __ATOMIC_ACQUIRE);
    if (err) return static_cast<ucclResult_t>(err);
    if (comm->abortFlag.load(std::memory_order_relaxed)) return ucclRemoteError;
    if ((++spins & 0xff) == 0) {
      if (nowMs() > dl) {
        commSetError(comm, "network %s with rank %d made no progress for %llu ms", c->isSend ? "send" : "receive",
                     c->peer, (unsigned long long)comm->cfg.waitTimeoutMs);
        {
          std::lock_guard<std::mutex> lk(comm->ctrMu);
          comm->counters.waitTimeouts++;
        }
        return ucclRemoteError;
      }
      sched_yield();
    }
  }
  return ucclSuccess;
}

ucclResult_t netHostAcquire(Comm* comm, NetConn* c, char** slot) {
  const uint64_t step = c->step;
  if (step >= UCCL_STEPS) {
    ucclResult_t r = hostSpin(comm, c, step - UCCL_STEPS + 1);
    if (r != ucclSuccess) return r;
  }
  if (slot) *slot = netSlot(c, step);
  return ucclSuccess;
}

ucclResult_t netHostPost(Comm* comm, NetConn* c, uint32_t op, size_t bytes, uint64_t* stepOut) {
  const uint64_t step = c->step;
  if (step >= UCCL_STEPS) {
    ucclResult_t r = hostSpin(comm, c, step - UCCL_STEPS + 1);  // slot reuse: wait for head > step - STEPS
    if (r != ucclSuccess) return r;
  }
  FifoEntry& e = c->fifo->entries[step % UCCL_STEPS];
  e.op = op;
  e.slot = static_cast<uint32_t>(step % UCCL_STEPS);
  e.bytes = bytes;
  e.step = step;
  e.result = 0;
  fifoStoreRelease(&c->fifo->tail, step + 1);
  c->step = step + 1;
  if (stepOut) *stepOut = step;
  return ucclSuccess;
}

ucclResult_t netHostWait(Comm* comm, NetConn* c, uint64_t step, size_t* bytesOut) {
  ucclResult_t r = hostSpin(comm, c, step + 1);
  if (r != ucclSuccess) return r;
  if (bytesOut) *bytesOut = static_cast<size_t>(c->fifo->entries[step % UCCL_STEPS].result);
  return ucclSuccess;
}

}  // namespace uccl
