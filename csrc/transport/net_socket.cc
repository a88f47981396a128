// Built-in network transport: tagged, framed messages over TCP sockets.
//
// Fills the plugin slot the way the reference's built-in UCX transport does
// (src/plugin/net_ucx.cc:110-516: listen / connect / accept handshake, tagged send and receive,
// request polling, progress entry point, force-close) but over plain sockets, so that the
// proxy path can be exercised between processes of one machine (loopback) as well as between
// machines.  Host pointers only: the caller stages device data through pinned bounce slots.
//
// Wire format per message: {u64 tag, u64 size} header followed by `size` payload bytes.
// Requests on one connection complete strictly in posting order.  isend/irecv never return a
// NULL request, even when the whole message moved inside the call.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <deque>
#include <mutex>
#include <set>
#include <string>

#include "../core/bootstrap.h"
#include "../core/log.h"
#include "net_plugin.h"

namespace uccl {
namespace {

struct SockCtx;

struct WireHeader {
  uint64_t tag;
  uint64_t size;
};

struct SockRequest {
  bool isSend = false;
  char* data = nullptr;
  size_t size = 0;        // send: bytes to send; recv: capacity
  WireHeader hdr = {0, 0};
  size_t hdrDone = 0;
  size_t done = 0;
  bool complete = false;
  bool failed = false;
  struct SockComm* comm = nullptr;
};

struct SockComm {
  SockCtx* ctx = nullptr;
  int fd = -1;
  bool isSend = false;
  uint64_t tag = 0;
  std::deque<SockRequest*> queue;  // posted, not yet complete, in order
  bool broken = false;
};

struct SockListen {
  SockCtx* ctx = nullptr;
  int fd = -1;
};

struct SockCtx {
  std::mutex mu;
  struct in_addr ip;
  std::set<SockComm*> comms;
};

void tuneSocket(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int sz = 4 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &sz, sizeof(sz));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &sz, sizeof(sz));
  int fl = fcntl(fd, F_GETFL, 0);
  if (fl >= 0) fcntl(fd, F_SETFL, fl | O_NONBLOCK);
}

// Moves as many bytes as the socket takes without blocking.  Returns false on a hard error.
bool pump(SockComm* c, SockRequest* r) {
  if (r->isSend) {
    while (r->hdrDone < sizeof(WireHeader)) {
      ssize_t n = ::send(c->fd, reinterpret_cast<char*>(&r->hdr) + r->hdrDone, sizeof(WireHeader) - r->hdrDone,
                         MSG_NOSIGNAL | MSG_DONTWAIT);
      if (n > 0) { r->hdrDone += n; continue; }
      if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) return true;
      return false;
    }
    while (r->done < r->size) {
      ssize_t n = ::send(c->fd, r->data + r->done, r->size - r->done, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (n > 0) { r->done += n; continue; }
      if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR)) return true;
      return false;
    }
    r->complete = true;
    return true;
  }
  while (r->hdrDone < sizeof(WireHeader)) {
    ssize_t n = ::recv(c->fd, reinterpret_cast<char*>(&r->hdr) + r->hdrDone, sizeof(WireHeader) - r->hdrDone,
                       MSG_DONTWAIT);
    if (n > 0) { r->hdrDone += n; continue; }
    if (n == 0) return false;
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return true;
    return false;
  }
  if (r->hdr.size > r->size) {
    UCCL_LOG(ERROR, "socket net: incoming message of %llu bytes exceeds the posted %zu",
             (unsigned long long)r->hdr.size, r->size);
    return false;
  }
  if (c->tag != 0 && r->hdr.tag != c->tag) {
    UCCL_LOG(ERROR, "socket net: tag mismatch (got %llx, expected %llx)", (unsigned long long)r->hdr.tag,
             (unsigned long long)c->tag);
    return false;
  }
  while (r->done < r->hdr.size) {
    ssize_t n = ::recv(c->fd, r->data + r->done, r->hdr.size - r->done, MSG_DONTWAIT);
    if (n > 0) { r->done += n; continue; }
    if (n == 0) return false;
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return true;
    return false;
  }
  r->complete = true;
  return true;
}

void progressComm(SockComm* c) {
  while (!c->queue.empty()) {
    SockRequest* r = c->queue.front();
    if (c->broken || !pump(c, r)) {
      c->broken = true;
      r->failed = true;
      r->complete = true;
    }
    if (!r->complete) break;
    c->queue.pop_front();
  }
}

// ------------------------------------------------------------------ v-table
ucclResult_t sockInit(void** handle) {
  if (!handle) return ucclInvalidArgument;
  SockCtx* ctx = new SockCtx();
  const char* ifn = getenv("UCCL_SOCKET_IFNAME");
  if (!ifn) ifn = getenv("UCCL_BOOTSTRAP_IFNAME");
  if (pickInterfaceAddr(ifn ? ifn : "", &ctx->ip) != 0) ctx->ip.s_addr = htonl(INADDR_LOOPBACK);
  *handle = ctx;
  return ucclSuccess;
}

ucclResult_t sockFinalize(void* handle) {
  SockCtx* ctx = static_cast<SockCtx*>(handle);
  if (!ctx) return ucclSuccess;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    for (SockComm* c : ctx->comms) {
      if (c->fd >= 0) ::close(c->fd);
      c->fd = -1;
      c->ctx = nullptr;
    }
    ctx->comms.clear();
  }
  delete ctx;
  return ucclSuccess;
}

ucclResult_t sockDevices(int* ndev) {
  if (!ndev) return ucclInvalidArgument;
  *ndev = 1;
  return ucclSuccess;
}

ucclResult_t sockGetProperties(int dev, ucclNetProperties_t* p) {
  if (!p || dev != 0) return ucclInvalidArgument;
  memset(p, 0, sizeof(*p));
  snprintf(p->name, sizeof(p->name), "Socket");
  p->ptrSupport = UCCL_PTR_HOST;
  p->speed = 12500;    // 100 Gb/s class NIC, MB/s
  p->latency = 20000;  // ns, kernel TCP stack
  p->maxComms = 65536;
  return ucclSuccess;
}

ucclResult_t sockListen(void* handle, void* listenAddr, void** listenComm) {
  SockCtx* ctx = static_cast<SockCtx*>(handle);
  if (!ctx || !listenAddr || !listenComm) return ucclInvalidArgument;
  int fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return ucclSystemError;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  struct sockaddr_in sa;
  memset(&sa, 0, sizeof(sa));
  sa.sin_family = AF_INET;
  sa.sin_addr.s_addr = htonl(INADDR_ANY);
  sa.sin_port = 0;
  if (bind(fd, reinterpret_cast<struct sockaddr*>(&sa), sizeof(sa)) != 0 || listen(fd, 256) != 0) {
    ::close(fd);
    return ucclSystemError;
  }
  socklen_t sl = sizeof(sa);
  getsockname(fd, reinterpret_cast<struct sockaddr*>(&sa), &sl);
  sa.sin_addr = ctx->ip;
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  memset(listenAddr, 0, UCCL_NET_HANDLE_BYTES);
  memcpy(listenAddr, &sa, sizeof(sa));
  SockListen* l = new SockListen();
  l->ctx = ctx;
  l->fd = fd;
  *listenComm = l;
  return ucclSuccess;
}

ucclResult_t sockConnect(void* handle, void* connectAddr, void** sendComm) {
  SockCtx* ctx = static_cast<SockCtx*>(handle);
  if (!ctx || !connectAddr || !sendComm) return ucclInvalidArgument;
  struct sockaddr_in sa;
  memcpy(&sa, connectAddr, sizeof(sa));
  const uint64_t dl = nowMs() + 30000;
  int fd = -1;
  while (true) {
    fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return ucclSystemError;
    if (connect(fd, reinterpret_cast<struct sockaddr*>(&sa), sizeof(sa)) == 0) break;
    ::close(fd);
    fd = -1;
    if (nowMs() > dl) return ucclRemoteError;
    usleep(10000);
  }
  tuneSocket(fd);
  SockComm* c = new SockComm();
  c->ctx = ctx;
  c->fd = fd;
  c->isSend = true;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->comms.insert(c);
  }
  *sendComm = c;
  return ucclSuccess;
}

ucclResult_t sockAccept(void* listenComm, void** recvComm) {
  SockListen* l = static_cast<SockListen*>(listenComm);
  if (!l || !recvComm) return ucclInvalidArgument;
  int fd = accept4(l->fd, nullptr, nullptr, SOCK_CLOEXEC);
  if (fd < 0) {
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return ucclInProgress;
    return ucclSystemError;
  }
  tuneSocket(fd);
  SockComm* c = new SockComm();
  c->ctx = l->ctx;
  c->fd = fd;
  c->isSend = false;
  {
    std::lock_guard<std::mutex> lk(l->ctx->mu);
    l->ctx->comms.insert(c);
  }
  *recvComm = c;
  return ucclSuccess;
}

ucclResult_t sockRegMr(void* comm, void* data, size_t size, int type, void** mhandle) {
  (void)comm; (void)size;
  if (!data || !mhandle) return ucclInvalidArgument;
  if (type != UCCL_PTR_HOST) return ucclInvalidArgument;  // no GPUDirect over TCP
  *mhandle = data;  // nothing to pin: any non-NULL cookie will do
  return ucclSuccess;
}
ucclResult_t sockDeregMr(void* comm, void* mhandle) {
  (void)comm; (void)mhandle;
  return ucclSuccess;
}

ucclResult_t sockPost(void* commV, void* data, size_t size, void** request, bool isSend) {
  SockComm* c = static_cast<SockComm*>(commV);
  if (!c || !request || (size && !data) || c->isSend != isSend) return ucclInvalidArgument;
  if (!c->ctx) return ucclInvalidUsage;
  std::lock_guard<std::mutex> lk(c->ctx->mu);
  if (c->broken) return ucclRemoteError;
  SockRequest* r = new SockRequest();
  r->isSend = isSend;
  r->data = static_cast<char*>(data);
  r->size = size;
  r->comm = c;
  if (isSend) r->hdr = {c->tag, size};
  c->queue.push_back(r);
  progressComm(c);
  *request = r;
  return ucclSuccess;
}
ucclResult_t sockIsend(void* c, void* d, size_t s, void* mh, void** req) { (void)mh; return sockPost(c, d, s, req, true); }
ucclResult_t sockIrecv(void* c, void* d, size_t s, void* mh, void** req) { (void)mh; return sockPost(c, d, s, req, false); }

ucclResult_t sockTest(void* request, int* done, int* size) {
  SockRequest* r = static_cast<SockRequest*>(request);
  if (!r || !done) return ucclInvalidArgument;
  SockComm* c = r->comm;
  if (!r->complete && c && c->ctx) {
    std::lock_guard<std::mutex> lk(c->ctx->mu);
    progressComm(c);
  }
  if (!r->complete) {
    *done = 0;
    return ucclSuccess;
  }
  *done = 1;
  if (size) *size = static_cast<int>(r->isSend ? r->size : r->hdr.size);
  const bool failed = r->failed;
  delete r;
  return failed ? ucclRemoteError : ucclSuccess;
}

ucclResult_t sockCloseComm(void* commV) {
  SockComm* c = static_cast<SockComm*>(commV);
  if (!c) return ucclSuccess;
  if (c->ctx) {
    std::lock_guard<std::mutex> lk(c->ctx->mu);
    c->ctx->comms.erase(c);
  }
  for (SockRequest* r : c->queue) delete r;
  if (c->fd >= 0) {
    shutdown(c->fd, SHUT_RDWR);
    ::close(c->fd);
  }
  delete c;
  return ucclSuccess;
}
ucclResult_t sockCloseListen(void* listenComm) {
  SockListen* l = static_cast<SockListen*>(listenComm);
  if (!l) return ucclSuccess;
  if (l->fd >= 0) ::close(l->fd);
  delete l;
  return ucclSuccess;
}

ucclResult_t sockProgress(void* handle) {
  SockCtx* ctx = static_cast<SockCtx*>(handle);
  if (!ctx) return ucclInvalidArgument;
  std::lock_guard<std::mutex> lk(ctx->mu);
  for (SockComm* c : ctx->comms) progressComm(c);
  return ucclSuccess;
}

ucclResult_t sockSetTag(void* commV, uint64_t tag) {
  SockComm* c = static_cast<SockComm*>(commV);
  if (!c) return ucclInvalidArgument;
  c->tag = tag;
  return ucclSuccess;
}

ucclNet_t g_socketPlugin = {
    "Socket",      sockInit,      sockFinalize,  sockDevices,   sockGetProperties, sockListen,
    sockConnect,   sockAccept,    sockRegMr,     sockDeregMr,   sockIsend,         sockIrecv,
    sockTest,      sockCloseComm, sockCloseComm, sockCloseListen, sockProgress,    sockSetTag};

}  // namespace

ucclNet_t* builtinSocketPlugin() { return &g_socketPlugin; }

}  // namespace uccl
