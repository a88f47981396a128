#include "bootstrap.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <random>
#include <thread>

#include "log.h"

namespace uccl {

namespace {

constexpr int kTagRing = -1;

struct RankHello {
  uint64_t magic;
  uint8_t nonce[16];
  int32_t rank;
  int32_t nranks;
  struct sockaddr_in addr;
};

struct PeerHello {
  uint64_t magic;
  int32_t src;
  int32_t tag;
  uint64_t size;
};

struct FdMsg {
  uint64_t magic;
  int32_t src;
  int32_t tag;
};

void setNoDelay(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}
void setNonBlocking(int fd, bool on) {
  int fl = fcntl(fd, F_GETFL, 0);
  if (fl < 0) return;
  fcntl(fd, F_SETFL, on ? (fl | O_NONBLOCK) : (fl & ~O_NONBLOCK));
}

// Blocking (with deadline) full read/write on a socket that may be in either mode.
bool xferAll(int fd, void* buf, size_t len, bool isSend, uint64_t deadlineMs,
             const std::atomic<uint32_t>* abortFlag) {
  char* p = static_cast<char*>(buf);
  size_t done = 0;
  while (done < len) {
    ssize_t n = isSend ? ::send(fd, p + done, len - done, MSG_NOSIGNAL | MSG_DONTWAIT)
                       : ::recv(fd, p + done, len - done, MSG_DONTWAIT);
    if (n > 0) {
      done += static_cast<size_t>(n);
      continue;
    }
    if (n == 0 && !isSend) return false;  // peer closed
    if (n < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return false;
    if (abortFlag && abortFlag->load(std::memory_order_relaxed)) return false;
    if (nowMs() > deadlineMs) return false;
    struct pollfd pfd = {fd, static_cast<short>(isSend ? POLLOUT : POLLIN), 0};
    poll(&pfd, 1, 50);
  }
  return true;
}

int tcpListen(struct in_addr bindAddr, int port, struct sockaddr_in* bound) {
  int fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -1;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  struct sockaddr_in sa;
  memset(&sa, 0, sizeof(sa));
  sa.sin_family = AF_INET;
  sa.sin_addr.s_addr = htonl(INADDR_ANY);
  sa.sin_port = htons(static_cast<uint16_t>(port));
  if (bind(fd, reinterpret_cast<struct sockaddr*>(&sa), sizeof(sa)) != 0 || listen(fd, 1024) != 0) {
    ::close(fd);
    return -1;
  }
  socklen_t sl = sizeof(sa);
  getsockname(fd, reinterpret_cast<struct sockaddr*>(&sa), &sl);
  sa.sin_addr = bindAddr;  // advertise the chosen interface address
  *bound = sa;
  return fd;
}

int tcpConnect(const struct sockaddr_in& to, uint64_t deadlineMs, const std::atomic<uint32_t>* abortFlag) {
  while (true) {
    int fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return -1;
    setNonBlocking(fd, true);
    int rc = connect(fd, reinterpret_cast<const struct sockaddr*>(&to), sizeof(to));
    if (rc != 0 && errno == EINPROGRESS) {
      while (true) {
        struct pollfd pfd = {fd, POLLOUT, 0};
        int pr = poll(&pfd, 1, 50);
        if (pr > 0) {
          int soerr = 0;
          socklen_t sl = sizeof(soerr);
          getsockopt(fd, SOL_SOCKET, SO_ERROR, &soerr, &sl);
          rc = soerr == 0 ? 0 : -1;
          errno = soerr;
          break;
        }
        if ((abortFlag && abortFlag->load(std::memory_order_relaxed)) || nowMs() > deadlineMs) {
          ::close(fd);
          return -1;
        }
      }
    }
    if (rc == 0) {
      setNoDelay(fd);
      return fd;
    }
    ::close(fd);
    // The peer may not be listening yet (root started later, or backlog full): retry.
    if ((abortFlag && abortFlag->load(std::memory_order_relaxed)) || nowMs() > deadlineMs) return -1;
    struct timespec ts = {0, 20 * 1000 * 1000};
    nanosleep(&ts, nullptr);
  }
}

void fillNonce(uint8_t* nonce) {
  std::random_device rd;
  std::mt19937_64 gen((static_cast<uint64_t>(rd()) << 32) ^ rd() ^ (static_cast<uint64_t>(getpid()) << 17) ^
                      static_cast<uint64_t>(nowMs()));
  for (int i = 0; i < 16; i += 8) {
    uint64_t v = gen();
    memcpy(nonce + i, &v, 8);
  }
}

// The rendezvous service: collect one hello per rank, answer with the address table.
void rootService(int listenFd, BootstrapIdPayload idp, uint64_t timeoutMs) {
  std::vector<int> fds;
  std::vector<struct sockaddr_in> table;
  int nranks = -1, got = 0;
  const uint64_t dl = nowMs() + timeoutMs;
  bool ok = true;
  while (ok && (nranks < 0 || got < nranks)) {
    struct pollfd pfd = {listenFd, POLLIN, 0};
    int pr = poll(&pfd, 1, 100);
    if (pr <= 0) {
      if (nowMs() > dl) ok = false;
      continue;
    }
    int c = accept4(listenFd, nullptr, nullptr, SOCK_CLOEXEC);
    if (c < 0) continue;
    setNoDelay(c);
    RankHello h;
    if (!xferAll(c, &h, sizeof(h), false, dl, nullptr) || h.magic != kBootstrapMagic ||
        memcmp(h.nonce, idp.nonce, 16) != 0 || h.nranks <= 0 || h.nranks > UCCL_MAX_RANKS || h.rank < 0 ||
        h.rank >= h.nranks) {
      ::close(c);  // stray connection: ignore
      continue;
    }
    if (nranks < 0) {
      nranks = h.nranks;
      fds.assign(nranks, -1);
      table.resize(nranks);
    }
    if (h.nranks != nranks || fds[h.rank] >= 0) {
      UCCL_LOG(ERROR, "bootstrap root: inconsistent hello from rank %d (nranks %d vs %d)", h.rank, h.nranks,
               nranks);
      ::close(c);
      ok = false;
      break;
    }
    fds[h.rank] = c;
    table[h.rank] = h.addr;
    ++got;
  }
  if (ok) {
    for (int r = 0; r < nranks; ++r)
      xferAll(fds[r], table.data(), sizeof(struct sockaddr_in) * nranks, true, dl, nullptr);
  } else {
    UCCL_LOG(WARN, "bootstrap root: rendezvous incomplete (%d of %d ranks) -- closing", got, nranks);
  }
  for (int fd : fds)
    if (fd >= 0) ::close(fd);
  ::close(listenFd);
}

}  // namespace

uint64_t nowMs() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return static_cast<uint64_t>(ts.tv_sec) * 1000ull + static_cast<uint64_t>(ts.tv_nsec) / 1000000ull;
}

int pickInterfaceAddr(const std::string& ifname, struct in_addr* out) {
  struct ifaddrs* ifa = nullptr;
  struct in_addr loop;
  loop.s_addr = htonl(INADDR_LOOPBACK);
  if (getifaddrs(&ifa) != 0) {
    *out = loop;
    return 0;
  }
  bool found = false;
  for (struct ifaddrs* p = ifa; p; p = p->ifa_next) {
    if (!p->ifa_addr || p->ifa_addr->sa_family != AF_INET) continue;
    if (!(p->ifa_flags & IFF_UP)) continue;
    const bool isLoop = (p->ifa_flags & IFF_LOOPBACK) != 0;
    if (!ifname.empty()) {
      if (ifname != p->ifa_name) continue;
    } else if (isLoop) {
      continue;
    }
    *out = reinterpret_cast<struct sockaddr_in*>(p->ifa_addr)->sin_addr;
    found = true;
    break;
  }
  freeifaddrs(ifa);
  if (!found) {
    if (!ifname.empty() && ifname != "lo") return -1;
    *out = loop;
  }
  return 0;
}

ucclResult_t bootstrapCreateRoot(ucclUniqueId* id, const Config& cfg) {
  if (!id) return ucclInvalidArgument;
  struct in_addr ip;
  if (pickInterfaceAddr(cfg.bootstrapIf, &ip) != 0) {
    UCCL_LOG(ERROR, "bootstrap: interface '%s' not found", cfg.bootstrapIf.c_str());
    return ucclSystemError;
  }
  BootstrapIdPayload p;
  memset(&p, 0, sizeof(p));
  p.magic = kBootstrapMagic;
  p.version = UCCL_VERSION;
  p.pid = static_cast<uint32_t>(getpid());
  fillNonce(p.nonce);
  int fd = tcpListen(ip, cfg.bootstrapPort, &p.addr);
  if (fd < 0) {
    UCCL_LOG(ERROR, "bootstrap: cannot listen on port %d: %s", cfg.bootstrapPort, strerror(errno));
    return ucclSystemError;
  }
  memcpy(id->internal, &p, sizeof(p));
  std::thread(rootService, fd, p, cfg.bootstrapTimeoutMs).detach();
  char buf[64];
  inet_ntop(AF_INET, &p.addr.sin_addr, buf, sizeof(buf));
  UCCL_LOG(INFO, "bootstrap root listening on %s:%d", buf, ntohs(p.addr.sin_port));
  return ucclSuccess;
}

ucclResult_t bootstrapIdFromAddress(const char* ip, int port, uint64_t seed, ucclUniqueId* id) {
  if (!ip || !id || port <= 0 || port > 65535) return ucclInvalidArgument;
  BootstrapIdPayload p;
  memset(&p, 0, sizeof(p));
  p.magic = kBootstrapMagic;
  p.version = UCCL_VERSION;
  p.pid = 0;
  std::mt19937_64 gen(seed ^ 0x9e3779b97f4a7c15ull);
  for (int i = 0; i < 16; i += 8) {
    uint64_t v = gen();
    memcpy(p.nonce + i, &v, 8);
  }
  p.addr.sin_family = AF_INET;
  p.addr.sin_port = htons(static_cast<uint16_t>(port));
  if (inet_pton(AF_INET, ip, &p.addr.sin_addr) != 1) return ucclInvalidArgument;
  memcpy(id->internal, &p, sizeof(p));
  return ucclSuccess;
}

ucclResult_t bootstrapServeId(const ucclUniqueId& id, const Config& cfg) {
  BootstrapIdPayload p;
  memcpy(&p, id.internal, sizeof(p));
  if (p.magic != kBootstrapMagic) return ucclInvalidArgument;
  struct sockaddr_in bound;
  int fd = tcpListen(p.addr.sin_addr, ntohs(p.addr.sin_port), &bound);
  if (fd < 0) {
    UCCL_LOG(ERROR, "bootstrap: cannot serve on port %d: %s", ntohs(p.addr.sin_port), strerror(errno));
    return ucclSystemError;
  }
  std::thread(rootService, fd, p, cfg.bootstrapTimeoutMs).detach();
  return ucclSuccess;
}

// ------------------------------------------------------------------ Bootstrap
Bootstrap::~Bootstrap() { close(); }

ucclResult_t Bootstrap::fail(ucclResult_t r, const char* fmt, ...) {
  char msg[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  err_ = msg;
  UCCL_LOG(ERROR, "bootstrap rank %d: %s", rank_, msg);
  return r;
}

uint64_t Bootstrap::deadline() const { return nowMs() + timeoutMs_; }
bool Bootstrap::expired(uint64_t dl) const {
  return nowMs() > dl || (abort_ && abort_->load(std::memory_order_relaxed));
}

ucclResult_t Bootstrap::ioAll(int fd, void* buf, size_t len, bool isSend, uint64_t dl) {
  return xferAll(fd, buf, len, isSend, dl, abort_) ? ucclSuccess : ucclRemoteError;
}

ucclResult_t Bootstrap::init(const ucclUniqueId& id, int rank, int nranks, const Config& cfg,
                             const std::atomic<uint32_t>* abortFlag) {
  rank_ = rank;
  nranks_ = nranks;
  abort_ = abortFlag;
  timeoutMs_ = cfg.bootstrapTimeoutMs;
  BootstrapIdPayload p;
  memcpy(&p, id.internal, sizeof(p));
  if (p.magic != kBootstrapMagic) return fail(ucclInvalidArgument, "unique id was not produced by ucclGetUniqueId");
  memcpy(nonce_, p.nonce, 16);
  if (nranks == 1) return ucclSuccess;

  const uint64_t dl = deadline();
  struct in_addr ip;
  if (pickInterfaceAddr(cfg.bootstrapIf, &ip) != 0) return fail(ucclSystemError, "interface not found");
  // If the root advertises loopback, everybody is on one host: stay on loopback too.
  if (ntohl(p.addr.sin_addr.s_addr) == INADDR_LOOPBACK) ip.s_addr = htonl(INADDR_LOOPBACK);
  struct sockaddr_in mine;
  listenFd_ = tcpListen(ip, 0, &mine);
  if (listenFd_ < 0) return fail(ucclSystemError, "listen failed: %s", strerror(errno));

  // abstract unix datagram socket for fd passing
  unixFd_ = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (unixFd_ >= 0) {
    struct sockaddr_un ua;
    memset(&ua, 0, sizeof(ua));
    ua.sun_family = AF_UNIX;
    char name[96];
    int n = snprintf(name, sizeof(name), "uccl-");
    for (int i = 0; i < 16; ++i) n += snprintf(name + n, sizeof(name) - n, "%02x", nonce_[i]);
    n += snprintf(name + n, sizeof(name) - n, "-%d", rank);
    memcpy(ua.sun_path + 1, name, n);
    if (bind(unixFd_, reinterpret_cast<struct sockaddr*>(&ua), offsetof(struct sockaddr_un, sun_path) + 1 + n) != 0) {
      UCCL_LOG(WARN, "bootstrap: unix socket bind failed: %s", strerror(errno));
      ::close(unixFd_);
      unixFd_ = -1;
    }
  }

  int rootFd = tcpConnect(p.addr, dl, abort_);
  if (rootFd < 0) return fail(ucclRemoteError, "cannot reach the rendezvous service: %s", strerror(errno));
  RankHello h;
  memset(&h, 0, sizeof(h));
  h.magic = kBootstrapMagic;
  memcpy(h.nonce, nonce_, 16);
  h.rank = rank;
  h.nranks = nranks;
  h.addr = mine;
  peers_.resize(nranks);
  ucclResult_t r = ioAll(rootFd, &h, sizeof(h), true, dl);
  if (r == ucclSuccess) r = ioAll(rootFd, peers_.data(), sizeof(struct sockaddr_in) * nranks, false, dl);
  ::close(rootFd);
  if (r != ucclSuccess) return fail(ucclRemoteError, "rendezvous failed (a rank is missing or the service timed out)");

  // ring: connect to next, accept from prev
  const int next = (rank + 1) % nranks, prev = (rank + nranks - 1) % nranks;
  nextFd_ = tcpConnect(peers_[next], dl, abort_);
  if (nextFd_ < 0) return fail(ucclRemoteError, "cannot connect to rank %d", next);
  PeerHello ph = {kBootstrapMagic, rank, kTagRing, 0};
  if (ioAll(nextFd_, &ph, sizeof(ph), true, dl) != ucclSuccess) return fail(ucclRemoteError, "ring hello failed");
  while (prevFd_ < 0) {
    int src, tag;
    uint64_t size;
    int fd = acceptOne(dl, &src, &tag, &size);
    if (fd < 0) return fail(ucclRemoteError, "rank %d never connected", prev);
    if (tag == kTagRing && src == prev) {
      prevFd_ = fd;
    } else {
      std::vector<uint8_t> buf(size);
      if (size && ioAll(fd, buf.data(), size, false, dl) != ucclSuccess) {
        ::close(fd);
        return fail(ucclRemoteError, "early message from rank %d truncated", src);
      }
      ::close(fd);
      stash_[{src, tag}].push_back(std::move(buf));
    }
  }
  return barrier();
}

int Bootstrap::acceptOne(uint64_t dl, int* srcRank, int* tag, uint64_t* size) {
  while (true) {
    struct pollfd pfd = {listenFd_, POLLIN, 0};
    int pr = poll(&pfd, 1, 50);
    if (pr > 0) {
      int c = accept4(listenFd_, nullptr, nullptr, SOCK_CLOEXEC);
      if (c < 0) continue;
      setNoDelay(c);
      PeerHello ph;
      if (!xferAll(c, &ph, sizeof(ph), false, dl, abort_) || ph.magic != kBootstrapMagic) {
        ::close(c);
        continue;
      }
      *srcRank = ph.src;
      *tag = ph.tag;
      *size = ph.size;
      return c;
    }
    if (expired(dl)) return -1;
  }
}

ucclResult_t Bootstrap::duplex(int sfd, const void* sbuf, int rfd, void* rbuf, size_t len, uint64_t dl) {
  size_t sd = 0, rd = 0;
  const char* sp = static_cast<const char*>(sbuf);
  char* rp = static_cast<char*>(rbuf);
  while (sd < len || rd < len) {
    bool moved = false;
    if (sd < len) {
      ssize_t n = ::send(sfd, sp + sd, len - sd, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (n > 0) { sd += n; moved = true; }
      else if (n < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return ucclRemoteError;
    }
    if (rd < len) {
      ssize_t n = ::recv(rfd, rp + rd, len - rd, MSG_DONTWAIT);
      if (n > 0) { rd += n; moved = true; }
      else if (n == 0) return ucclRemoteError;
      else if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) return ucclRemoteError;
    }
    if (!moved) {
      if (expired(dl)) return ucclRemoteError;
      struct pollfd pfds[2] = {{sfd, static_cast<short>(sd < len ? POLLOUT : 0), 0},
                               {rfd, static_cast<short>(rd < len ? POLLIN : 0), 0}};
      poll(pfds, 2, 20);
    }
  }
  return ucclSuccess;
}

ucclResult_t Bootstrap::allGather(void* data, size_t bytes) {
  if (nranks_ <= 1 || bytes == 0) return ucclSuccess;
  char* d = static_cast<char*>(data);
  const uint64_t dl = deadline();
  for (int s = 0; s < nranks_ - 1; ++s) {
    const int sendSlot = (rank_ - s + nranks_) % nranks_;
    const int recvSlot = (rank_ - s - 1 + nranks_) % nranks_;
    ucclResult_t r = duplex(nextFd_, d + sendSlot * bytes, prevFd_, d + recvSlot * bytes, bytes, dl);
    if (r != ucclSuccess) return fail(r, "all-gather step %d failed (peer gone or timeout)", s);
  }
  return ucclSuccess;
}

ucclResult_t Bootstrap::barrier() {
  if (nranks_ <= 1) return ucclSuccess;
  std::vector<uint8_t> tok(nranks_, 0);
  tok[rank_] = 1;
  return allGather(tok.data(), 1);
}

ucclResult_t Bootstrap::send(int peer, int tag, const void* data, size_t bytes) {
  if (peer < 0 || peer >= nranks_ || tag < 0) return ucclInvalidArgument;
  if (peer == rank_) {
    std::vector<uint8_t> buf(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + bytes);
    stash_[{peer, tag}].push_back(std::move(buf));
    return ucclSuccess;
  }
  const uint64_t dl = deadline();
  int fd = tcpConnect(peers_[peer], dl, abort_);
  if (fd < 0) return fail(ucclRemoteError, "send: cannot connect to rank %d", peer);
  PeerHello ph = {kBootstrapMagic, rank_, tag, bytes};
  ucclResult_t r = ioAll(fd, &ph, sizeof(ph), true, dl);
  if (r == ucclSuccess && bytes) r = ioAll(fd, const_cast<void*>(data), bytes, true, dl);
  // No acknowledgement: the payload (control-plane sized, far below the socket buffer) is
  // delivered before the FIN, and two ranks that send to each other first cannot deadlock.
  ::close(fd);
  if (r != ucclSuccess) return fail(r, "send to rank %d failed", peer);
  return ucclSuccess;
}

ucclResult_t Bootstrap::recv(int peer, int tag, void* data, size_t bytes) {
  if (peer < 0 || peer >= nranks_ || tag < 0) return ucclInvalidArgument;
  const uint64_t dl = deadline();
  while (true) {
    auto it = stash_.find({peer, tag});
    if (it != stash_.end() && !it->second.empty()) {
      std::vector<uint8_t> buf = std::move(it->second.front());
      it->second.erase(it->second.begin());
      if (buf.size() != bytes) return fail(ucclInternalError, "recv size mismatch from rank %d", peer);
      if (bytes) memcpy(data, buf.data(), bytes);
      return ucclSuccess;
    }
    int src, t;
    uint64_t size;
    int fd = acceptOne(dl, &src, &t, &size);
    if (fd < 0) return fail(ucclRemoteError, "recv from rank %d tag %d timed out", peer, tag);
    std::vector<uint8_t> buf(size);
    ucclResult_t r = size ? ioAll(fd, buf.data(), size, false, dl) : ucclSuccess;
    ::close(fd);
    if (r != ucclSuccess) return fail(r, "message from rank %d truncated", src);
    stash_[{src, t}].push_back(std::move(buf));
  }
}

static void unixPeerAddr(const uint8_t* nonce, int rank, struct sockaddr_un* ua, socklen_t* len) {
  memset(ua, 0, sizeof(*ua));
  ua->sun_family = AF_UNIX;
  char name[96];
  int n = snprintf(name, sizeof(name), "uccl-");
  for (int i = 0; i < 16; ++i) n += snprintf(name + n, sizeof(name) - n, "%02x", nonce[i]);
  n += snprintf(name + n, sizeof(name) - n, "-%d", rank);
  memcpy(ua->sun_path + 1, name, n);
  *len = static_cast<socklen_t>(offsetof(struct sockaddr_un, sun_path) + 1 + n);
}

ucclResult_t Bootstrap::sendFd(int peer, int tag, int fd) {
  if (unixFd_ < 0) return fail(ucclSystemError, "fd passing unavailable (unix socket not bound)");
  struct sockaddr_un ua;
  socklen_t ul;
  unixPeerAddr(nonce_, peer, &ua, &ul);
  FdMsg m = {kBootstrapMagic, rank_, tag};
  struct iovec iov = {&m, sizeof(m)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  struct msghdr mh;
  memset(&mh, 0, sizeof(mh));
  mh.msg_name = &ua;
  mh.msg_namelen = ul;
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  mh.msg_control = ctrl;
  mh.msg_controllen = sizeof(ctrl);
  struct cmsghdr* cm = CMSG_FIRSTHDR(&mh);
  cm->cmsg_level = SOL_SOCKET;
  cm->cmsg_type = SCM_RIGHTS;
  cm->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(cm), &fd, sizeof(int));
  const uint64_t dl = deadline();
  while (true) {
    ssize_t n = sendmsg(unixFd_, &mh, MSG_NOSIGNAL | MSG_DONTWAIT);
    if (n == static_cast<ssize_t>(sizeof(m))) return ucclSuccess;
    if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR || errno == ECONNREFUSED ||
                  errno == ENOBUFS)) {
      if (expired(dl)) return fail(ucclRemoteError, "sendFd to rank %d timed out", peer);
      struct timespec ts = {0, 2 * 1000 * 1000};
      nanosleep(&ts, nullptr);
      continue;
    }
    return fail(ucclSystemError, "sendFd to rank %d: %s", peer, strerror(errno));
  }
}

ucclResult_t Bootstrap::recvFd(int peer, int tag, int* fd) {
  if (unixFd_ < 0) return fail(ucclSystemError, "fd passing unavailable (unix socket not bound)");
  const uint64_t dl = deadline();
  while (true) {
    auto it = fdStash_.find({peer, tag});
    if (it != fdStash_.end() && !it->second.empty()) {
      *fd = it->second.front();
      it->second.erase(it->second.begin());
      return ucclSuccess;
    }
    struct pollfd pfd = {unixFd_, POLLIN, 0};
    int pr = poll(&pfd, 1, 50);
    if (pr <= 0) {
      if (expired(dl)) return fail(ucclRemoteError, "recvFd from rank %d tag %d timed out", peer, tag);
      continue;
    }
    FdMsg m;
    struct iovec iov = {&m, sizeof(m)};
    char ctrl[CMSG_SPACE(sizeof(int))];
    struct msghdr mh;
    memset(&mh, 0, sizeof(mh));
    mh.msg_iov = &iov;
    mh.msg_iovlen = 1;
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    ssize_t n = recvmsg(unixFd_, &mh, MSG_DONTWAIT | MSG_CMSG_CLOEXEC);
    if (n != static_cast<ssize_t>(sizeof(m)) || m.magic != kBootstrapMagic) continue;
    struct cmsghdr* cm = CMSG_FIRSTHDR(&mh);
    if (!cm || cm->cmsg_level != SOL_SOCKET || cm->cmsg_type != SCM_RIGHTS) continue;
    int got;
    memcpy(&got, CMSG_DATA(cm), sizeof(int));
    fdStash_[{m.src, m.tag}].push_back(got);
  }
}

void Bootstrap::close() {
  if (nextFd_ >= 0) ::close(nextFd_);
  if (prevFd_ >= 0 && prevFd_ != nextFd_) ::close(prevFd_);
  if (listenFd_ >= 0) ::close(listenFd_);
  if (unixFd_ >= 0) ::close(unixFd_);
  for (auto& kv : fdStash_)
    for (int fd : kv.second) ::close(fd);
  fdStash_.clear();
  nextFd_ = prevFd_ = listenFd_ = unixFd_ = -1;
}

}  // namespace uccl
