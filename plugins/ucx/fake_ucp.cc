// Test stand-in for the UCP calls that plugins/ucx/plugin.cc uses (see fake_ucp/ucp/api/ucp.h):
// tagged messages over non-blocking TCP sockets, driven entirely by ucp_worker_progress().
//
// Semantics kept from UCX, because the plugin relies on them: a tagged send may complete inline
// (NULL status pointer) or hand back a request; receives are posted on the worker and match on
// (tag & mask); messages that arrive before their receive is posted are buffered ("unexpected")
// and matched in arrival order; connection requests reach the listener's callback from inside
// progress; a forced endpoint close never waits for the peer.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <string.h>
#include <sys/socket.h>
#include <ucp/api/ucp.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <deque>
#include <mutex>
#include <set>
#include <vector>

namespace {

struct Hdr {
  uint64_t tag;
  uint64_t len;
};

struct Request {
  ucs_status_t status = UCS_INPROGRESS;
  size_t length = 0;
  ucp_tag_t tag = 0;
  // posted receive
  char* buf = nullptr;
  size_t cap = 0;
  ucp_tag_t want = 0, mask = 0;
  bool released = false;  // ucp_request_free came before completion
};

struct SendOp {
  Hdr hdr;
  const char* data;
  size_t done = 0;  // bytes of header + payload written
  Request* req = nullptr;
};

struct Unexpected {
  ucp_tag_t tag;
  std::vector<char> data;
};

std::atomic<int> g_registrations{0};

void nonblock(int fd) {
  const int fl = fcntl(fd, F_GETFL, 0);
  if (fl >= 0) fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}
bool again() { return errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR; }

}  // namespace

struct ucp_config {};
struct ucp_context {};
struct ucp_mem {};
struct ucp_conn_request {
  int fd;
};

struct ucp_ep {
  ucp_worker_h worker = nullptr;
  int fd = -1;
  bool broken = false;
  std::deque<SendOp> sends;
  // incoming message being assembled
  Hdr inHdr = {0, 0};
  size_t inHdrDone = 0, inDone = 0;
  Request* inReq = nullptr;     // matched posted receive, or
  std::vector<char> inTemp;     // temporary storage of an unexpected message
  bool inActive = false;
};

struct ucp_listener {
  ucp_worker_h worker = nullptr;
  int fd = -1;
  ucp_listener_conn_handler_t handler = {nullptr, nullptr};
};

struct ucp_worker {
  std::recursive_mutex mu;
  std::set<ucp_ep*> eps;
  std::set<ucp_listener*> listeners;
  std::deque<Request*> posted;
  std::deque<Unexpected> unexpected;
};

namespace {

void finish(Request* r, ucs_status_t st) {
  r->status = st;
  if (r->released) delete r;
}

unsigned progressSends(ucp_ep* ep) {
  unsigned n = 0;
  while (!ep->sends.empty() && !ep->broken) {
    SendOp& op = ep->sends.front();
    const size_t total = sizeof(Hdr) + op.hdr.len;
    while (op.done < total) {
      const char* p;
      size_t left;
      if (op.done < sizeof(Hdr)) {
        p = reinterpret_cast<const char*>(&op.hdr) + op.done;
        left = sizeof(Hdr) - op.done;
      } else {
        p = op.data + (op.done - sizeof(Hdr));
        left = total - op.done;
      }
      const ssize_t w = send(ep->fd, p, left, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (w > 0) {
        op.done += static_cast<size_t>(w);
        ++n;
      } else if (w < 0 && again()) {
        return n;
      } else {
        ep->broken = true;
        break;
      }
    }
    if (ep->broken) break;
    if (op.req) finish(op.req, UCS_OK);
    ep->sends.pop_front();
  }
  if (ep->broken) {
    for (SendOp& op : ep->sends)
      if (op.req) finish(op.req, UCS_ERR_CONNECTION_RESET);
    ep->sends.clear();
  }
  return n;
}

unsigned progressRecv(ucp_ep* ep) {
  ucp_worker* w = ep->worker;
  unsigned n = 0;
  while (!ep->broken) {
    if (ep->inHdrDone < sizeof(Hdr)) {
      const ssize_t r = recv(ep->fd, reinterpret_cast<char*>(&ep->inHdr) + ep->inHdrDone, sizeof(Hdr) - ep->inHdrDone, MSG_DONTWAIT);
      if (r > 0) {
        ep->inHdrDone += static_cast<size_t>(r);
        ++n;
        if (ep->inHdrDone < sizeof(Hdr)) continue;
        // header complete: a posted receive takes the payload directly, else it is buffered
        ep->inDone = 0;
        ep->inReq = nullptr;
        ep->inActive = true;
        for (auto it = w->posted.begin(); it != w->posted.end(); ++it)
          if (((*it)->want & (*it)->mask) == (ep->inHdr.tag & (*it)->mask)) {
            ep->inReq = *it;
            w->posted.erase(it);
            break;
          }
        if (!ep->inReq) ep->inTemp.assign(ep->inHdr.len, 0);
      } else if (r == 0) {
        ep->broken = true;  // orderly shutdown by the peer: nothing more will arrive
        break;
      } else if (again()) {
        break;
      } else {
        ep->broken = true;
        break;
      }
    }
    if (ep->inHdrDone == sizeof(Hdr)) {
      const size_t len = ep->inHdr.len;
      bool stalled = false;
      while (ep->inDone < len) {
        char scratch[4096];
        char* dst;
        size_t room = len - ep->inDone;
        if (ep->inReq) {
          if (ep->inDone < ep->inReq->cap) {
            dst = ep->inReq->buf + ep->inDone;
            room = std::min(room, ep->inReq->cap - ep->inDone);
          } else {  // truncated: drain the rest
            dst = scratch;
            room = std::min(room, sizeof(scratch));
          }
        } else {
          dst = ep->inTemp.data() + ep->inDone;
        }
        const ssize_t r = recv(ep->fd, dst, room, MSG_DONTWAIT);
        if (r > 0) {
          ep->inDone += static_cast<size_t>(r);
          ++n;
        } else if (r < 0 && again()) {
          stalled = true;
          break;
        } else {
          ep->broken = true;
          break;
        }
      }
      if (ep->broken || stalled) break;
      if (ep->inReq) {
        ep->inReq->length = std::min(len, ep->inReq->cap);
        ep->inReq->tag = ep->inHdr.tag;
        finish(ep->inReq, len > ep->inReq->cap ? UCS_ERR_MESSAGE_TRUNCATED : UCS_OK);
      } else {
        // a receive may have been posted while this message was still arriving
        Request* late = nullptr;
        for (auto it = w->posted.begin(); it != w->posted.end(); ++it)
          if (((*it)->want & (*it)->mask) == (ep->inHdr.tag & (*it)->mask)) {
            late = *it;
            w->posted.erase(it);
            break;
          }
        if (late) {
          memcpy(late->buf, ep->inTemp.data(), std::min(len, late->cap));
          late->length = std::min(len, late->cap);
          late->tag = ep->inHdr.tag;
          finish(late, len > late->cap ? UCS_ERR_MESSAGE_TRUNCATED : UCS_OK);
        } else {
          w->unexpected.push_back({ep->inHdr.tag, std::move(ep->inTemp)});
        }
        ep->inTemp.clear();
      }
      ep->inReq = nullptr;
      ep->inActive = false;
      ep->inHdrDone = 0;
    }
  }
  if (ep->broken && ep->inActive && ep->inReq) {
    finish(ep->inReq, UCS_ERR_CONNECTION_RESET);
    ep->inReq = nullptr;
    ep->inActive = false;
  }
  return n;
}

}  // namespace

extern "C" {

const char* ucs_status_string(ucs_status_t s) {
  switch (s) {
    case UCS_OK: return "Success";
    case UCS_INPROGRESS: return "Operation in progress";
    case UCS_ERR_NO_MEMORY: return "Out of memory";
    case UCS_ERR_INVALID_PARAM: return "Invalid parameter";
    case UCS_ERR_UNREACHABLE: return "Destination is unreachable";
    case UCS_ERR_MESSAGE_TRUNCATED: return "Message truncated";
    case UCS_ERR_CONNECTION_RESET: return "Connection reset by remote peer";
    default: return "Unknown error";
  }
}

ucs_status_t ucp_config_read(const char*, const char*, ucp_config_t** out) {
  *out = new ucp_config();
  return UCS_OK;
}
void ucp_config_release(ucp_config_t* c) { delete c; }

ucs_status_t ucp_init(const ucp_params_t* p, const ucp_config_t*, ucp_context_h* out) {
  if (!p || !(p->field_mask & UCP_PARAM_FIELD_FEATURES) || !(p->features & UCP_FEATURE_TAG)) return UCS_ERR_INVALID_PARAM;
  *out = new ucp_context();
  return UCS_OK;
}
void ucp_cleanup(ucp_context_h c) { delete c; }

ucs_status_t ucp_worker_create(ucp_context_h c, const ucp_worker_params_t*, ucp_worker_h* out) {
  if (!c) return UCS_ERR_INVALID_PARAM;
  *out = new ucp_worker();
  return UCS_OK;
}
void ucp_worker_destroy(ucp_worker_h w) {
  if (!w) return;
  for (ucp_ep* e : w->eps) {
    if (e->fd >= 0) close(e->fd);
    delete e;
  }
  for (Request* r : w->posted) delete r;
  delete w;
}

unsigned ucp_worker_progress(ucp_worker_h w) {
  std::lock_guard<std::recursive_mutex> lk(w->mu);
  unsigned n = 0;
  for (ucp_listener* l : w->listeners) {
    for (;;) {
      const int fd = accept(l->fd, nullptr, nullptr);
      if (fd < 0) break;
      nonblock(fd);
      ucp_conn_request* req = new ucp_conn_request{fd};
      if (l->handler.cb) l->handler.cb(req, l->handler.arg);
      ++n;
    }
  }
  for (ucp_ep* e : w->eps) {
    n += progressSends(e);
    n += progressRecv(e);
  }
  return n;
}

ucs_status_t ucp_listener_create(ucp_worker_h w, const ucp_listener_params_t* p, ucp_listener_h* out) {
  if (!w || !p || !(p->field_mask & UCP_LISTENER_PARAM_FIELD_SOCK_ADDR)) return UCS_ERR_INVALID_PARAM;
  const int fd = socket(p->sockaddr.addr->sa_family, SOCK_STREAM, 0);
  if (fd < 0) return UCS_ERR_UNREACHABLE;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  if (bind(fd, p->sockaddr.addr, p->sockaddr.addrlen) != 0 || listen(fd, 128) != 0) {
    close(fd);
    return UCS_ERR_UNREACHABLE;
  }
  const int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  ucp_listener* l = new ucp_listener();
  l->worker = w;
  l->fd = fd;
  if (p->field_mask & UCP_LISTENER_PARAM_FIELD_CONN_HANDLER) l->handler = p->conn_handler;
  std::lock_guard<std::recursive_mutex> lk(w->mu);
  w->listeners.insert(l);
  *out = l;
  return UCS_OK;
}

ucs_status_t ucp_listener_query(ucp_listener_h l, ucp_listener_attr_t* attr) {
  if (!l || !attr || !(attr->field_mask & UCP_LISTENER_ATTR_FIELD_SOCKADDR)) return UCS_ERR_INVALID_PARAM;
  socklen_t len = sizeof(attr->sockaddr);
  memset(&attr->sockaddr, 0, sizeof(attr->sockaddr));
  return getsockname(l->fd, reinterpret_cast<sockaddr*>(&attr->sockaddr), &len) == 0 ? UCS_OK : UCS_ERR_UNREACHABLE;
}

void ucp_listener_destroy(ucp_listener_h l) {
  if (!l) return;
  {
    std::lock_guard<std::recursive_mutex> lk(l->worker->mu);
    l->worker->listeners.erase(l);
  }
  close(l->fd);
  delete l;
}

ucs_status_t ucp_ep_create(ucp_worker_h w, const ucp_ep_params_t* p, ucp_ep_h* out) {
  if (!w || !p) return UCS_ERR_INVALID_PARAM;
  int fd = -1;
  if (p->field_mask & UCP_EP_PARAM_FIELD_CONN_REQUEST) {
    fd = p->conn_request->fd;
    delete p->conn_request;
  } else if (p->field_mask & UCP_EP_PARAM_FIELD_SOCK_ADDR) {
    fd = socket(p->sockaddr.addr->sa_family, SOCK_STREAM, 0);
    if (fd < 0) return UCS_ERR_UNREACHABLE;
    if (connect(fd, p->sockaddr.addr, p->sockaddr.addrlen) != 0) {
      close(fd);
      return UCS_ERR_UNREACHABLE;
    }
    nonblock(fd);
  } else {
    return UCS_ERR_INVALID_PARAM;
  }
  ucp_ep* e = new ucp_ep();
  e->worker = w;
  e->fd = fd;
  std::lock_guard<std::recursive_mutex> lk(w->mu);
  w->eps.insert(e);
  *out = e;
  return UCS_OK;
}

ucs_status_ptr_t ucp_ep_close_nbx(ucp_ep_h e, const ucp_request_param_t*) {
  if (!e) return nullptr;
  ucp_worker* w = e->worker;
  std::lock_guard<std::recursive_mutex> lk(w->mu);
  e->broken = true;
  progressSends(e);  // fails what is still queued
  if (e->inActive && e->inReq) finish(e->inReq, UCS_ERR_CONNECTION_RESET);
  w->eps.erase(e);
  if (e->fd >= 0) close(e->fd);
  delete e;
  return nullptr;
}

ucs_status_ptr_t ucp_tag_send_nbx(ucp_ep_h e, const void* buf, size_t count, ucp_tag_t tag, const ucp_request_param_t*) {
  if (!e) return UCS_STATUS_PTR(UCS_ERR_INVALID_PARAM);
  std::lock_guard<std::recursive_mutex> lk(e->worker->mu);
  if (e->broken) return UCS_STATUS_PTR(UCS_ERR_CONNECTION_RESET);
  SendOp op;
  op.hdr = {tag, count};
  op.data = static_cast<const char*>(buf);
  e->sends.push_back(op);
  SendOp* mine = &e->sends.back();
  progressSends(e);
  if (e->broken) return UCS_STATUS_PTR(UCS_ERR_CONNECTION_RESET);
  // `mine` is still queued exactly when the queue is non-empty and its last entry is this one
  if (e->sends.empty() || &e->sends.back() != mine) return nullptr;  // went out inline
  Request* r = new Request();
  e->sends.back().req = r;
  return r;
}

ucs_status_ptr_t ucp_tag_recv_nbx(ucp_worker_h w, void* buf, size_t count, ucp_tag_t tag, ucp_tag_t mask,
                                  const ucp_request_param_t*) {
  if (!w) return UCS_STATUS_PTR(UCS_ERR_INVALID_PARAM);
  std::lock_guard<std::recursive_mutex> lk(w->mu);
  Request* r = new Request();
  r->buf = static_cast<char*>(buf);
  r->cap = count;
  r->want = tag;
  r->mask = mask;
  for (auto it = w->unexpected.begin(); it != w->unexpected.end(); ++it)
    if ((it->tag & mask) == (tag & mask)) {
      const size_t len = it->data.size();
      memcpy(r->buf, it->data.data(), std::min(len, count));
      r->length = std::min(len, count);
      r->tag = it->tag;
      r->status = len > count ? UCS_ERR_MESSAGE_TRUNCATED : UCS_OK;
      w->unexpected.erase(it);
      return r;
    }
  w->posted.push_back(r);
  return r;
}

ucs_status_t ucp_request_check_status(void* request) { return static_cast<Request*>(request)->status; }

ucs_status_t ucp_tag_recv_request_test(void* request, ucp_tag_recv_info_t* info) {
  Request* r = static_cast<Request*>(request);
  if (r->status == UCS_OK && info) {
    info->length = r->length;
    info->sender_tag = r->tag;
  }
  return r->status;
}

void ucp_request_free(void* request) {
  Request* r = static_cast<Request*>(request);
  if (r->status == UCS_INPROGRESS) r->released = true;  // still owned by a queue
  else delete r;
}

ucs_status_t ucp_mem_map(ucp_context_h c, const ucp_mem_map_params_t* p, ucp_mem_h* out) {
  if (!c || !p || !(p->field_mask & UCP_MEM_MAP_PARAM_FIELD_ADDRESS) || !(p->field_mask & UCP_MEM_MAP_PARAM_FIELD_LENGTH) ||
      !p->address || !p->length)
    return UCS_ERR_INVALID_PARAM;
  *out = new ucp_mem();
  g_registrations.fetch_add(1);
  return UCS_OK;
}
ucs_status_t ucp_mem_unmap(ucp_context_h, ucp_mem_h m) {
  if (!m) return UCS_ERR_INVALID_PARAM;
  delete m;
  g_registrations.fetch_sub(1);
  return UCS_OK;
}

int fake_ucp_live_registrations(void) { return g_registrations.load(); }

}  // extern "C"
