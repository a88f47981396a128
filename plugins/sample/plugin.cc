// Sample external network plugin: libuccl-net-sample.so exporting `ucclNetPlugin_v1`.
//
// Shows the dlopen ABI end to end.  Unlike the reference's sample (plugins/ucx/plugin.cc:180-199,
// whose isend/irecv mark a request complete without moving a byte), this one is a working
// transport: messages travel over abstract-namespace AF_UNIX stream sockets, so it connects
// processes of one host.  Load it with UCCL_NET_PLUGIN=/path/to/libuccl-net-sample.so.
// It depends on nothing but libc and the two public headers.
#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <deque>
#include <mutex>
#include <set>

#include "uccl_net.h"

namespace {

struct Ctx;
struct Req;

struct Hdr {
  uint64_t tag;
  uint64_t size;
};

struct Comm {
  Ctx* ctx = nullptr;
  int fd = -1;
  bool sender = false;
  uint64_t tag = 0;
  bool broken = false;
  std::deque<Req*> q;
};

struct Req {
  Comm* comm = nullptr;
  char* data = nullptr;
  size_t cap = 0;
  Hdr hdr = {0, 0};
  size_t hdrDone = 0, done = 0;
  bool complete = false, failed = false;
};

struct Listen {
  Ctx* ctx = nullptr;
  int fd = -1;
};

struct Ctx {
  std::mutex mu;
  std::set<Comm*> comms;
};

std::atomic<uint64_t> g_listenSeq{0};

void nonblock(int fd) {
  int fl = fcntl(fd, F_GETFL, 0);
  if (fl >= 0) fcntl(fd, F_SETFL, fl | O_NONBLOCK);
}

bool again() { return errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR; }

bool step(Comm* c, Req* r) {
  if (c->sender) {
    while (r->hdrDone < sizeof(Hdr)) {
      ssize_t n = send(c->fd, (char*)&r->hdr + r->hdrDone, sizeof(Hdr) - r->hdrDone, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (n > 0) r->hdrDone += n;
      else return n < 0 && again();
    }
    while (r->done < r->hdr.size) {
      ssize_t n = send(c->fd, r->data + r->done, r->hdr.size - r->done, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (n > 0) r->done += n;
      else return n < 0 && again();
    }
  } else {
    while (r->hdrDone < sizeof(Hdr)) {
      ssize_t n = recv(c->fd, (char*)&r->hdr + r->hdrDone, sizeof(Hdr) - r->hdrDone, MSG_DONTWAIT);
      if (n > 0) r->hdrDone += n;
      else return n < 0 && again();
    }
    if (r->hdr.size > r->cap || (c->tag && r->hdr.tag != c->tag)) return false;
    while (r->done < r->hdr.size) {
      ssize_t n = recv(c->fd, r->data + r->done, r->hdr.size - r->done, MSG_DONTWAIT);
      if (n > 0) r->done += n;
      else return n < 0 && again();
    }
  }
  r->complete = true;
  return true;
}

void drive(Comm* c) {
  while (!c->q.empty()) {
    Req* r = c->q.front();
    if (c->broken || !step(c, r)) {
      c->broken = true;
      r->failed = r->complete = true;
    }
    if (!r->complete) return;
    c->q.pop_front();
  }
}

ucclResult_t pInit(void** h) {
  if (!h) return ucclInvalidArgument;
  *h = new Ctx();
  return ucclSuccess;
}
ucclResult_t pFinalize(void* h) {
  delete static_cast<Ctx*>(h);
  return ucclSuccess;
}
ucclResult_t pDevices(int* n) {
  if (!n) return ucclInvalidArgument;
  *n = 1;
  return ucclSuccess;
}
ucclResult_t pProps(int dev, ucclNetProperties_t* p) {
  if (dev != 0 || !p) return ucclInvalidArgument;
  memset(p, 0, sizeof(*p));
  snprintf(p->name, sizeof(p->name), "UnixSample");
  p->ptrSupport = UCCL_PTR_HOST;
  p->speed = 5000;
  p->latency = 5000;
  p->maxComms = 4096;
  return ucclSuccess;
}
ucclResult_t pListen(void* h, void* addr, void** lc) {
  if (!h || !addr || !lc) return ucclInvalidArgument;
  int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return ucclSystemError;
  struct sockaddr_un ua;
  memset(&ua, 0, sizeof(ua));
  ua.sun_family = AF_UNIX;
  int n = snprintf(ua.sun_path + 1, sizeof(ua.sun_path) - 1, "uccl-sample-%d-%llu", (int)getpid(),
                   (unsigned long long)g_listenSeq.fetch_add(1));
  socklen_t len = (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + n);
  if (bind(fd, (struct sockaddr*)&ua, len) != 0 || listen(fd, 64) != 0) {
    close(fd);
    return ucclSystemError;
  }
  nonblock(fd);
  memset(addr, 0, UCCL_NET_HANDLE_BYTES);
  memcpy(addr, &len, sizeof(len));
  memcpy((char*)addr + sizeof(len), &ua, len);
  Listen* l = new Listen();
  l->ctx = static_cast<Ctx*>(h);
  l->fd = fd;
  *lc = l;
  return ucclSuccess;
}
Comm* newComm(Ctx* ctx, int fd, bool sender) {
  nonblock(fd);
  Comm* c = new Comm();
  c->ctx = ctx;
  c->fd = fd;
  c->sender = sender;
  std::lock_guard<std::mutex> lk(ctx->mu);
  ctx->comms.insert(c);
  return c;
}
ucclResult_t pConnect(void* h, void* addr, void** sc) {
  if (!h || !addr || !sc) return ucclInvalidArgument;
  socklen_t len;
  memcpy(&len, addr, sizeof(len));
  struct sockaddr_un ua;
  memset(&ua, 0, sizeof(ua));
  if (len > sizeof(ua)) return ucclInvalidArgument;
  memcpy(&ua, (char*)addr + sizeof(len), len);
  int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return ucclSystemError;
  for (int attempt = 0; connect(fd, (struct sockaddr*)&ua, len) != 0; ++attempt) {
    if (attempt > 3000) {
      close(fd);
      return ucclRemoteError;
    }
    usleep(10000);
  }
  *sc = newComm(static_cast<Ctx*>(h), fd, true);
  return ucclSuccess;
}
ucclResult_t pAccept(void* lc, void** rc) {
  Listen* l = static_cast<Listen*>(lc);
  if (!l || !rc) return ucclInvalidArgument;
  int fd = accept4(l->fd, nullptr, nullptr, SOCK_CLOEXEC);
  if (fd < 0) return again() ? ucclInProgress : ucclSystemError;
  *rc = newComm(l->ctx, fd, false);
  return ucclSuccess;
}
ucclResult_t pRegMr(void*, void* data, size_t, int type, void** mh) {
  if (!data || !mh || type != UCCL_PTR_HOST) return ucclInvalidArgument;
  *mh = data;
  return ucclSuccess;
}
ucclResult_t pDeregMr(void*, void*) { return ucclSuccess; }
ucclResult_t post(void* cv, void* data, size_t size, void** req, bool sender) {
  Comm* c = static_cast<Comm*>(cv);
  if (!c || !req || c->sender != sender || (size && !data)) return ucclInvalidArgument;
  std::lock_guard<std::mutex> lk(c->ctx->mu);
  if (c->broken) return ucclRemoteError;
  Req* r = new Req();
  r->comm = c;
  r->data = static_cast<char*>(data);
  r->cap = size;
  if (sender) r->hdr = {c->tag, size};
  c->q.push_back(r);
  drive(c);
  *req = r;
  return ucclSuccess;
}
ucclResult_t pIsend(void* c, void* d, size_t s, void*, void** r) { return post(c, d, s, r, true); }
ucclResult_t pIrecv(void* c, void* d, size_t s, void*, void** r) { return post(c, d, s, r, false); }
ucclResult_t pTest(void* rv, int* done, int* size) {
  Req* r = static_cast<Req*>(rv);
  if (!r || !done) return ucclInvalidArgument;
  if (!r->complete) {
    std::lock_guard<std::mutex> lk(r->comm->ctx->mu);
    drive(r->comm);
  }
  *done = r->complete ? 1 : 0;
  if (!r->complete) return ucclSuccess;
  if (size) *size = (int)r->hdr.size;
  bool failed = r->failed;
  delete r;
  return failed ? ucclRemoteError : ucclSuccess;
}
ucclResult_t pClose(void* cv) {
  Comm* c = static_cast<Comm*>(cv);
  if (!c) return ucclSuccess;
  {
    std::lock_guard<std::mutex> lk(c->ctx->mu);
    c->ctx->comms.erase(c);
  }
  for (Req* r : c->q) delete r;
  if (c->fd >= 0) close(c->fd);
  delete c;
  return ucclSuccess;
}
ucclResult_t pCloseListen(void* lc) {
  Listen* l = static_cast<Listen*>(lc);
  if (!l) return ucclSuccess;
  if (l->fd >= 0) close(l->fd);
  delete l;
  return ucclSuccess;
}
ucclResult_t pProgress(void* h) {
  Ctx* ctx = static_cast<Ctx*>(h);
  if (!ctx) return ucclInvalidArgument;
  std::lock_guard<std::mutex> lk(ctx->mu);
  for (Comm* c : ctx->comms) drive(c);
  return ucclSuccess;
}
ucclResult_t pSetTag(void* cv, uint64_t tag) {
  if (!cv) return ucclInvalidArgument;
  static_cast<Comm*>(cv)->tag = tag;
  return ucclSuccess;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) ucclNet_t ucclNetPlugin_v1 = {
    "UnixSample", pInit,  pFinalize, pDevices, pProps,  pListen, pConnect,     pAccept,   pRegMr,
    pDeregMr,     pIsend, pIrecv,    pTest,    pClose,  pClose,  pCloseListen, pProgress, pSetTag};
