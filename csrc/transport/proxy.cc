// Proxy thread: the only caller of the network plugin's data-path functions.
//
// Same division of labour as the reference's proxy (src/proxy.cc:26-164): producers describe work
// in FIFOs, this thread posts isend/irecv, polls test() and publishes completions in order.  The
// differences: completion is published through a monotonic `head` counter instead of per-entry
// flags; whether an entry has been posted is tracked in proxy-private state (`posted`), never by
// a NULL request pointer, so an operation that finishes inside isend()/irecv() is not posted a
// second time; plugin errors are latched into the FIFO's error word, the communicator's
// asynchronous error and the device-visible abort word; and a heartbeat counter lets the owner
// check that the thread is alive.
#include <sched.h>
#include <time.h>

#include "../core/comm.h"
#include "../core/log.h"

namespace uccl {

ucclResult_t proxyProgressConn(ucclNet_t* net, NetConn* c, uint64_t* posts, uint64_t* completions) {
  ConnFifo* f = c->fifo;
  if (!f || !c->netComm) return ucclSuccess;
  if (__atomic_load_n(&f->error, __ATOMIC_RELAXED)) return ucclSuccess;  // latched: nothing more to do
  const uint64_t tail = fifoLoadAcquire(&f->tail);
  uint64_t head = f->head;  // only this thread writes it

  while (c->posted < tail) {
    const int idx = static_cast<int>(c->posted % UCCL_STEPS);
    FifoEntry& e = f->entries[idx];
    const uint32_t slot = e.slot % UCCL_STEPS;
    char* ptr = c->bounce + static_cast<size_t>(slot) * c->slotBytes;
    void* req = nullptr;
    ucclResult_t r;
    switch (e.op) {
      case FIFO_SEND:
      case FIFO_PUT:
        r = net->isend(c->netComm, ptr, e.bytes, c->mhandle[slot], &req);
        break;
      case FIFO_RECV:
      case FIFO_WAIT:
        r = net->irecv(c->netComm, ptr, e.bytes ? e.bytes : c->slotBytes, c->mhandle[slot], &req);
        break;
      case FIFO_SIGNAL:
        r = net->isend(c->netComm, ptr, 0, c->mhandle[slot], &req);
        break;
      default:
        r = ucclInternalError;
        break;
    }
    if (r == ucclInProgress) break;  // plugin is out of resources: retry on the next pass
    if (r != ucclSuccess || req == nullptr) {
      const ucclResult_t err = r != ucclSuccess ? r : ucclInternalError;
      __atomic_store_n(&f->error, static_cast<uint64_t>(err), __ATOMIC_RELEASE);
      return err;
    }
    c->request[idx] = req;
    ++c->posted;
    if (posts) ++*posts;
  }

  while (head < c->posted) {
    const int idx = static_cast<int>(head % UCCL_STEPS);
    int done = 0, size = 0;
    ucclResult_t r = net->test(c->request[idx], &done, &size);
    if (r != ucclSuccess) {
      c->request[idx] = nullptr;
      __atomic_store_n(&f->error, static_cast<uint64_t>(r), __ATOMIC_RELEASE);
      return r;
    }
    if (!done) break;  // strict in-order completion
    c->request[idx] = nullptr;
    f->entries[idx].result = static_cast<uint64_t>(size);
    ++head;
    fifoStoreRelease(&f->head, head);
    if (completions) ++*completions;
  }
  return ucclSuccess;
}

static void proxyMain(Comm* comm) {
  ProxyState& st = comm->proxy;
  st.running.store(true, std::memory_order_release);
  uint32_t idle = 0;
  std::vector<NetConn*> conns;
  while (!st.stop.load(std::memory_order_acquire)) {
    if (comm->abortFlag.load(std::memory_order_relaxed)) break;
    {
      std::lock_guard<std::mutex> lk(comm->netMu);
      conns = comm->allConns;
    }
    uint64_t posts = 0, completions = 0;
    for (NetConn* c : conns) {
      jitterPause(comm->cfg.jitterUs);
      ucclResult_t r = proxyProgressConn(comm->net, c, &posts, &completions);
      if (r != ucclSuccess) {
        commSetError(comm, "network %s to/from rank %d failed: %s", c->isSend ? "send" : "receive", c->peer,
                     ucclGetErrorString(r));
        commSetAsyncError(comm, r == ucclRemoteError ? ucclRemoteError : ucclSystemError);
        if (comm->hostFlags) __atomic_store_n(&comm->hostFlags[0], 1u, __ATOMIC_RELEASE);
      }
    }
    if (comm->net && comm->netContext) comm->net->progress(comm->netContext);
    st.heartbeat.fetch_add(1, std::memory_order_relaxed);
    if (posts) st.posts.fetch_add(posts, std::memory_order_relaxed);
    if (completions) st.completions.fetch_add(completions, std::memory_order_relaxed);
    if (posts == 0 && completions == 0) {
      if (++idle > 2000) {
        struct timespec ts = {0, 20000};
        nanosleep(&ts, nullptr);
      } else {
        sched_yield();
      }
    } else {
      idle = 0;
    }
  }
  st.running.store(false, std::memory_order_release);
}

ucclResult_t proxyStart(Comm* comm) {
  if (comm->proxy.thread.joinable()) return ucclSuccess;
  if (!comm->net) return ucclSuccess;  // nothing to drive
  comm->proxy.stop.store(false);
  try {
    comm->proxy.thread = std::thread(proxyMain, comm);
  } catch (...) {
    commSetError(comm, "cannot start the proxy thread");
    return ucclSystemError;
  }
  return ucclSuccess;
}

void proxyStop(Comm* comm) {
  comm->proxy.stop.store(true, std::memory_order_release);
  if (comm->proxy.thread.joinable()) comm->proxy.thread.join();
}

}  // namespace uccl
