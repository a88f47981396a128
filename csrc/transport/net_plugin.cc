// Plugin loader.  Same contract as the reference's loader (src/plugin/net_ucx.cc:580-652):
// environment override first, path sanity checks, dlopen + dlsym of `ucclNetPlugin_v1`, and a
// silent fall back to the built-in transport.  The built-in transport here is TCP sockets
// (net_socket.cc) because UCX is not part of the target image.
#include "net_plugin.h"

#include <dlfcn.h>
#include <string.h>

#include "../core/log.h"

namespace uccl {

bool netPluginComplete(const ucclNet_t* n, std::string* why) {
  if (!n) { if (why) *why = "null table"; return false; }
#define UCCL_NEED(field)                                             \
  if (!n->field) {                                                   \
    if (why) *why = std::string("plugin slot '") + #field + "' is empty"; \
    return false;                                                    \
  }
  UCCL_NEED(name) UCCL_NEED(init) UCCL_NEED(finalize) UCCL_NEED(devices) UCCL_NEED(getProperties)
  UCCL_NEED(listen) UCCL_NEED(connect) UCCL_NEED(accept) UCCL_NEED(regMr) UCCL_NEED(deregMr)
  UCCL_NEED(isend) UCCL_NEED(irecv) UCCL_NEED(test) UCCL_NEED(closeSend) UCCL_NEED(closeRecv)
  UCCL_NEED(closeListen) UCCL_NEED(progress) UCCL_NEED(setTag)
#undef UCCL_NEED
  return true;
}

ucclNet_t* loadNetPlugin(const std::string& path, std::string* why) {
  auto fail = [&](const std::string& m) -> ucclNet_t* {
    if (why) *why = m;
    UCCL_LOG(WARN, "net plugin '%s' rejected: %s", path.c_str(), m.c_str());
    return nullptr;
  };
  if (path.empty()) return fail("empty path");
  if (path.find("..") != std::string::npos) return fail("path must not contain '..'");
  if (path.size() < 4 || path.compare(path.size() - 3, 3, ".so") != 0) return fail("path must end in .so");
  void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!h) return fail(std::string("dlopen: ") + dlerror());
  void* sym = dlsym(h, UCCL_NET_PLUGIN_SYMBOL);
  if (!sym) {
    dlclose(h);
    return fail("symbol " UCCL_NET_PLUGIN_SYMBOL " not found");
  }
  ucclNet_t* net = static_cast<ucclNet_t*>(sym);
  std::string w;
  if (!netPluginComplete(net, &w)) {
    dlclose(h);
    return fail(w);
  }
  // The handle is intentionally kept open for the life of the process: communicators may
  // still hold function pointers into it.
  UCCL_LOG(INFO, "loaded net plugin '%s' from %s", net->name, path.c_str());
  return net;
}

ucclNet_t* autoLoadNetPlugin(const std::string& cfgPath) {
  if (!cfgPath.empty()) {
    std::string why;
    if (ucclNet_t* n = loadNetPlugin(cfgPath, &why)) return n;
    UCCL_LOG(WARN, "falling back to the built-in socket transport");
  }
  return builtinSocketPlugin();
}

}  // namespace uccl
