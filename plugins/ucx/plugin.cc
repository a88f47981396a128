// UCX transport plugin: libuccl-net-ucx.so exporting `ucclNetPlugin_v1`.
//
// Carries the network path over UCP tagged messages, which is what the reference's built-in
// transport does (src/plugin/net_ucx.cc:110-516): one UCP context and worker per plugin instance,
// a sockaddr listener whose connection requests are queued for accept(), client / server
// endpoints, ucp_tag_send_nbx / ucp_tag_recv_nbx with the 64-bit tag that setTag() assigned to the
// connection, ucp_mem_map registration (host or CUDA memory), forced endpoint close.
//
// UCX is not part of every image, so the file has two faces:
//   -DUCCL_HAS_UCX=1   the transport below, built against <ucp/api/ucp.h> (the real library, or
//                      the small stand-in under plugins/ucx/fake_ucp/ that the CPU tests use);
//   otherwise          a plugin whose init() reports that UCX support was not compiled in, the
//                      same role as the reference's no-UCX stubs (net_ucx.cc:518-546).
// Load with UCCL_NET_PLUGIN=/path/to/libuccl-net-ucx.so.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "uccl_net.h"

#if defined(UCCL_HAS_UCX) && UCCL_HAS_UCX

#include <arpa/inet.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <sys/socket.h>
#include <ucp/api/ucp.h>

#include <deque>
#include <mutex>
#include <new>

namespace {

struct Ctx {
  ucp_context_h context = nullptr;
  ucp_worker_h worker = nullptr;
  std::mutex mu;  // UCP runs in multi-thread mode; this guards the plugin's own queues
};

struct Listener {
  Ctx* ctx = nullptr;
  ucp_listener_h handle = nullptr;
  std::deque<ucp_conn_request_h> pending;  // filled by the connection handler, drained by accept()
};

struct Conn {
  Ctx* ctx = nullptr;
  ucp_ep_h ep = nullptr;
  uint64_t tag = 0;
  bool failed = false;
};

// One outstanding operation.  UCP hands back either a request pointer (still running), NULL
// (finished inline) or an error; the caller always gets a Req so that "posted" and "not posted"
// stay distinguishable.
struct Req {
  Ctx* ctx = nullptr;
  void* ucpReq = nullptr;  // nullptr: completed inline
  bool isRecv = false;
  size_t size = 0;         // bytes asked for (send) or capacity (receive)
  ucs_status_t inlineStatus = UCS_OK;
};

struct MemHandle {
  Ctx* ctx = nullptr;
  ucp_mem_h memh = nullptr;
};

// address the listener binds to and advertises: the interface named by UCCL_SOCKET_IFNAME, else
// the first interface that is up and not loopback, else loopback
bool pickAddress(sockaddr_in* out) {
  memset(out, 0, sizeof(*out));
  out->sin_family = AF_INET;
  out->sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  const char* want = getenv("UCCL_SOCKET_IFNAME");
  ifaddrs* list = nullptr;
  if (getifaddrs(&list) != 0) return true;
  bool found = false;
  for (int pass = 0; pass < 2 && !found; ++pass)
    for (ifaddrs* i = list; i && !found; i = i->ifa_next) {
      if (!i->ifa_addr || i->ifa_addr->sa_family != AF_INET || !(i->ifa_flags & IFF_UP)) continue;
      const bool loop = (i->ifa_flags & IFF_LOOPBACK) != 0;
      if (want && *want ? strcmp(want, i->ifa_name) != 0 : (pass == 0 ? loop : !loop)) continue;
      out->sin_addr = reinterpret_cast<sockaddr_in*>(i->ifa_addr)->sin_addr;
      found = true;
    }
  freeifaddrs(list);
  return true;
}

void onConnRequest(ucp_conn_request_h req, void* arg) {
  Listener* l = static_cast<Listener*>(arg);
  std::lock_guard<std::mutex> lk(l->ctx->mu);
  l->pending.push_back(req);
}

ucclResult_t ucxInit(void** handle) {
  if (!handle) return ucclInvalidArgument;
  Ctx* c = new (std::nothrow) Ctx();
  if (!c) return ucclSystemError;
  ucp_params_t params;
  memset(&params, 0, sizeof(params));
  params.field_mask = UCP_PARAM_FIELD_FEATURES;
  params.features = UCP_FEATURE_TAG | UCP_FEATURE_RMA | UCP_FEATURE_STREAM;
  ucp_config_t* config = nullptr;
  if (ucp_config_read(nullptr, nullptr, &config) != UCS_OK) config = nullptr;
  ucs_status_t st = ucp_init(&params, config, &c->context);
  if (config) ucp_config_release(config);
  if (st != UCS_OK) {
    fprintf(stderr, "uccl-net-ucx: ucp_init failed: %s\n", ucs_status_string(st));
    delete c;
    return ucclSystemError;
  }
  ucp_worker_params_t wp;
  memset(&wp, 0, sizeof(wp));
  wp.field_mask = UCP_WORKER_PARAM_FIELD_THREAD_MODE;
  wp.thread_mode = UCS_THREAD_MODE_MULTI;
  st = ucp_worker_create(c->context, &wp, &c->worker);
  if (st != UCS_OK) {
    fprintf(stderr, "uccl-net-ucx: ucp_worker_create failed: %s\n", ucs_status_string(st));
    ucp_cleanup(c->context);
    delete c;
    return ucclSystemError;
  }
  *handle = c;
  return ucclSuccess;
}

ucclResult_t ucxFinalize(void* handle) {
  Ctx* c = static_cast<Ctx*>(handle);
  if (!c) return ucclSuccess;
  if (c->worker) ucp_worker_destroy(c->worker);
  if (c->context) ucp_cleanup(c->context);
  delete c;
  return ucclSuccess;
}

ucclResult_t ucxDevices(int* ndev) {
  if (!ndev) return ucclInvalidArgument;
  *ndev = 1;  // UCP picks the transports and devices itself
  return ucclSuccess;
}

ucclResult_t ucxGetProperties(int dev, ucclNetProperties_t* p) {
  if (dev != 0 || !p) return ucclInvalidArgument;
  memset(p, 0, sizeof(*p));
  snprintf(p->name, sizeof(p->name), "UCX");
  p->ptrSupport = UCCL_PTR_HOST | UCCL_PTR_DEVICE;  // ucp_mem_map takes CUDA memory when UCX has CUDA support
  p->speed = 25000;    // MB/s placeholder: UCP does not expose link speed
  p->latency = 1000;   // ns
  p->maxComms = 65536;
  return ucclSuccess;
}

ucclResult_t ucxListen(void* handle, void* listenAddr, void** listenComm) {
  Ctx* c = static_cast<Ctx*>(handle);
  if (!c || !listenAddr || !listenComm) return ucclInvalidArgument;
  Listener* l = new (std::nothrow) Listener();
  if (!l) return ucclSystemError;
  l->ctx = c;
  sockaddr_in addr;
  pickAddress(&addr);
  addr.sin_port = 0;  // any free port
  ucp_listener_params_t lp;
  memset(&lp, 0, sizeof(lp));
  lp.field_mask = UCP_LISTENER_PARAM_FIELD_SOCK_ADDR | UCP_LISTENER_PARAM_FIELD_CONN_HANDLER;
  lp.sockaddr.addr = reinterpret_cast<const sockaddr*>(&addr);
  lp.sockaddr.addrlen = sizeof(addr);
  lp.conn_handler.cb = onConnRequest;
  lp.conn_handler.arg = l;
  ucs_status_t st = ucp_listener_create(c->worker, &lp, &l->handle);
  if (st != UCS_OK) {
    fprintf(stderr, "uccl-net-ucx: ucp_listener_create failed: %s\n", ucs_status_string(st));
    delete l;
    return ucclSystemError;
  }
  // the blob a peer passes to connect(): the address the listener really got
  ucp_listener_attr_t attr;
  memset(&attr, 0, sizeof(attr));
  attr.field_mask = UCP_LISTENER_ATTR_FIELD_SOCKADDR;
  st = ucp_listener_query(l->handle, &attr);
  if (st != UCS_OK) {
    ucp_listener_destroy(l->handle);
    delete l;
    return ucclSystemError;
  }
  static_assert(sizeof(sockaddr_storage) <= UCCL_NET_HANDLE_BYTES, "address blob too small");
  memset(listenAddr, 0, UCCL_NET_HANDLE_BYTES);
  memcpy(listenAddr, &attr.sockaddr, sizeof(sockaddr_storage));
  *listenComm = l;
  return ucclSuccess;
}

ucclResult_t ucxConnect(void* handle, void* connectAddr, void** sendComm) {
  Ctx* c = static_cast<Ctx*>(handle);
  if (!c || !connectAddr || !sendComm) return ucclInvalidArgument;
  Conn* s = new (std::nothrow) Conn();
  if (!s) return ucclSystemError;
  s->ctx = c;
  sockaddr_storage ss;
  memcpy(&ss, connectAddr, sizeof(ss));
  ucp_ep_params_t ep;
  memset(&ep, 0, sizeof(ep));
  ep.field_mask = UCP_EP_PARAM_FIELD_FLAGS | UCP_EP_PARAM_FIELD_SOCK_ADDR | UCP_EP_PARAM_FIELD_ERR_HANDLING_MODE;
  ep.flags = UCP_EP_PARAMS_FLAGS_CLIENT_SERVER;
  ep.err_mode = UCP_ERR_HANDLING_MODE_PEER;
  ep.sockaddr.addr = reinterpret_cast<const sockaddr*>(&ss);
  ep.sockaddr.addrlen = ss.ss_family == AF_INET6 ? sizeof(sockaddr_in6) : sizeof(sockaddr_in);
  ucs_status_t st = ucp_ep_create(c->worker, &ep, &s->ep);
  if (st != UCS_OK) {
    fprintf(stderr, "uccl-net-ucx: ucp_ep_create (client) failed: %s\n", ucs_status_string(st));
    delete s;
    return ucclSystemError;
  }
  *sendComm = s;
  return ucclSuccess;
}

ucclResult_t ucxAccept(void* listenComm, void** recvComm) {
  Listener* l = static_cast<Listener*>(listenComm);
  if (!l || !recvComm) return ucclInvalidArgument;
  ucp_worker_progress(l->ctx->worker);  // connection requests arrive through progress
  ucp_conn_request_h req = nullptr;
  {
    std::lock_guard<std::mutex> lk(l->ctx->mu);
    if (l->pending.empty()) return ucclInProgress;
    req = l->pending.front();
    l->pending.pop_front();
  }
  Conn* r = new (std::nothrow) Conn();
  if (!r) return ucclSystemError;
  r->ctx = l->ctx;
  ucp_ep_params_t ep;
  memset(&ep, 0, sizeof(ep));
  ep.field_mask = UCP_EP_PARAM_FIELD_CONN_REQUEST | UCP_EP_PARAM_FIELD_ERR_HANDLING_MODE;
  ep.err_mode = UCP_ERR_HANDLING_MODE_PEER;
  ep.conn_request = req;
  ucs_status_t st = ucp_ep_create(l->ctx->worker, &ep, &r->ep);
  if (st != UCS_OK) {
    fprintf(stderr, "uccl-net-ucx: ucp_ep_create (server) failed: %s\n", ucs_status_string(st));
    delete r;
    return ucclSystemError;
  }
  *recvComm = r;
  return ucclSuccess;
}

ucclResult_t ucxRegMr(void* comm, void* data, size_t size, int type, void** mhandle) {
  Conn* c = static_cast<Conn*>(comm);
  if (!c || !data || !size || !mhandle) return ucclInvalidArgument;
  MemHandle* m = new (std::nothrow) MemHandle();
  if (!m) return ucclSystemError;
  m->ctx = c->ctx;
  ucp_mem_map_params_t mp;
  memset(&mp, 0, sizeof(mp));
  mp.field_mask = UCP_MEM_MAP_PARAM_FIELD_ADDRESS | UCP_MEM_MAP_PARAM_FIELD_LENGTH | UCP_MEM_MAP_PARAM_FIELD_MEMORY_TYPE;
  mp.address = data;
  mp.length = size;
  // the reference leaves the memory type out (net_ucx.cc:313-346); say which it is
  mp.memory_type = (type & UCCL_PTR_DEVICE) ? UCS_MEMORY_TYPE_CUDA : UCS_MEMORY_TYPE_HOST;
  ucs_status_t st = ucp_mem_map(c->ctx->context, &mp, &m->memh);
  if (st != UCS_OK) {
    fprintf(stderr, "uccl-net-ucx: ucp_mem_map failed: %s\n", ucs_status_string(st));
    delete m;
    return ucclSystemError;
  }
  *mhandle = m;
  return ucclSuccess;
}

ucclResult_t ucxDeregMr(void* /*comm*/, void* mhandle) {
  MemHandle* m = static_cast<MemHandle*>(mhandle);
  if (!m) return ucclSuccess;
  if (m->memh) ucp_mem_unmap(m->ctx->context, m->memh);
  delete m;
  return ucclSuccess;
}

ucclResult_t finishPost(Conn* c, ucs_status_ptr_t sp, bool isRecv, size_t size, void** request) {
  if (UCS_PTR_IS_ERR(sp)) {
    c->failed = true;
    fprintf(stderr, "uccl-net-ucx: tagged %s failed: %s\n", isRecv ? "receive" : "send", ucs_status_string(UCS_PTR_STATUS(sp)));
    return ucclRemoteError;
  }
  Req* r = new (std::nothrow) Req();
  if (!r) return ucclSystemError;
  r->ctx = c->ctx;
  r->isRecv = isRecv;
  r->size = size;
  r->ucpReq = UCS_PTR_IS_PTR(sp) ? sp : nullptr;
  *request = r;
  return ucclSuccess;
}

ucclResult_t ucxIsend(void* sendComm, void* data, size_t size, void* /*mhandle*/, void** request) {
  Conn* c = static_cast<Conn*>(sendComm);
  if (!c || !request || (size && !data)) return ucclInvalidArgument;
  if (c->failed) return ucclRemoteError;
  ucp_request_param_t p;
  memset(&p, 0, sizeof(p));
  p.op_attr_mask = 0;  // contiguous bytes, no callback: completion is polled by test()
  return finishPost(c, ucp_tag_send_nbx(c->ep, data, size, c->tag, &p), false, size, request);
}

ucclResult_t ucxIrecv(void* recvComm, void* data, size_t size, void* /*mhandle*/, void** request) {
  Conn* c = static_cast<Conn*>(recvComm);
  if (!c || !request || (size && !data)) return ucclInvalidArgument;
  if (c->failed) return ucclRemoteError;
  ucp_request_param_t p;
  memset(&p, 0, sizeof(p));
  p.op_attr_mask = 0;
  // exact tag match: the tag names (source rank, destination rank, channel)
  return finishPost(c, ucp_tag_recv_nbx(c->ctx->worker, data, size, c->tag, ~0ull, &p), true, size, request);
}

ucclResult_t ucxTest(void* request, int* done, int* size) {
  Req* r = static_cast<Req*>(request);
  if (!r || !done) return ucclInvalidArgument;
  *done = 0;
  if (r->ucpReq == nullptr) {  // finished when it was posted
    *done = 1;
    if (size) *size = static_cast<int>(r->size);
    delete r;
    return ucclSuccess;
  }
  ucs_status_t st;
  size_t got = r->size;
  if (r->isRecv) {
    ucp_tag_recv_info_t info;
    memset(&info, 0, sizeof(info));
    st = ucp_tag_recv_request_test(r->ucpReq, &info);
    if (st == UCS_OK) got = info.length;
  } else {
    st = ucp_request_check_status(r->ucpReq);
  }
  if (st == UCS_INPROGRESS) {
    ucp_worker_progress(r->ctx->worker);
    return ucclSuccess;
  }
  ucp_request_free(r->ucpReq);
  const bool ok = st == UCS_OK;
  if (ok) {
    *done = 1;
    if (size) *size = static_cast<int>(got);
  } else {
    fprintf(stderr, "uccl-net-ucx: request failed: %s\n", ucs_status_string(st));
  }
  delete r;
  return ok ? ucclSuccess : ucclRemoteError;
}

ucclResult_t closeConn(void* comm) {
  Conn* c = static_cast<Conn*>(comm);
  if (!c) return ucclSuccess;
  if (c->ep) {
    // forced close: teardown must not wait for a peer that may be gone (net_ucx.cc:453-492)
    ucp_request_param_t p;
    memset(&p, 0, sizeof(p));
    p.op_attr_mask = UCP_OP_ATTR_FIELD_FLAGS;
    p.flags = UCP_EP_CLOSE_FLAG_FORCE;
    ucs_status_ptr_t sp = ucp_ep_close_nbx(c->ep, &p);
    if (UCS_PTR_IS_PTR(sp)) {
      for (int i = 0; i < 100000 && ucp_request_check_status(sp) == UCS_INPROGRESS; ++i) ucp_worker_progress(c->ctx->worker);
      ucp_request_free(sp);
    }
  }
  delete c;
  return ucclSuccess;
}

ucclResult_t ucxCloseListen(void* listenComm) {
  Listener* l = static_cast<Listener*>(listenComm);
  if (!l) return ucclSuccess;
  if (l->handle) ucp_listener_destroy(l->handle);
  delete l;
  return ucclSuccess;
}

ucclResult_t ucxProgress(void* handle) {
  Ctx* c = static_cast<Ctx*>(handle);
  if (c && c->worker) ucp_worker_progress(c->worker);
  return ucclSuccess;
}

ucclResult_t ucxSetTag(void* comm, uint64_t tag) {
  Conn* c = static_cast<Conn*>(comm);
  if (!c) return ucclInvalidArgument;
  c->tag = tag;
  return ucclSuccess;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) ucclNet_t ucclNetPlugin_v1 = {
    "UCX",        ucxInit,  ucxFinalize, ucxDevices, ucxGetProperties, ucxListen,  ucxConnect,     ucxAccept,   ucxRegMr,
    ucxDeregMr,   ucxIsend, ucxIrecv,    ucxTest,    closeConn,        closeConn,  ucxCloseListen, ucxProgress, ucxSetTag,
};

#else  // ---------------------------------------------------------------- built without UCX

namespace {

ucclResult_t noUcxInit(void** handle) {
  if (handle) *handle = nullptr;
  fprintf(stderr, "uccl-net-ucx: built without UCX support (rebuild with UCCL_BUILD_UCX_PLUGIN=1 UCX_HOME=<prefix>)\n");
  return ucclInvalidUsage;
}
ucclResult_t noUcxFinalize(void*) { return ucclSuccess; }
ucclResult_t noUcxDevices(int* ndev) {
  if (ndev) *ndev = 0;
  return ucclSuccess;
}
ucclResult_t noUcxProps(int, ucclNetProperties_t*) { return ucclInvalidUsage; }
ucclResult_t noUcxListen(void*, void*, void**) { return ucclInvalidUsage; }
ucclResult_t noUcxConnect(void*, void*, void**) { return ucclInvalidUsage; }
ucclResult_t noUcxAccept(void*, void**) { return ucclInvalidUsage; }
ucclResult_t noUcxRegMr(void*, void*, size_t, int, void**) { return ucclInvalidUsage; }
ucclResult_t noUcxDeregMr(void*, void*) { return ucclSuccess; }
ucclResult_t noUcxPost(void*, void*, size_t, void*, void**) { return ucclInvalidUsage; }
ucclResult_t noUcxTest(void*, int*, int*) { return ucclInvalidUsage; }
ucclResult_t noUcxClose(void*) { return ucclSuccess; }
ucclResult_t noUcxProgress(void*) { return ucclSuccess; }
ucclResult_t noUcxSetTag(void*, uint64_t) { return ucclInvalidUsage; }

}  // namespace

extern "C" __attribute__((visibility("default"))) ucclNet_t ucclNetPlugin_v1 = {
    "UCX (not compiled in)", noUcxInit,  noUcxFinalize, noUcxDevices, noUcxProps, noUcxListen, noUcxConnect,
    noUcxAccept,             noUcxRegMr, noUcxDeregMr,  noUcxPost,    noUcxPost,  noUcxTest,   noUcxClose,
    noUcxClose,              noUcxClose, noUcxProgress, noUcxSetTag,
};

#endif
