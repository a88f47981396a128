// Network plugin discovery: built-in TCP socket transport, optional external shared object.
#pragma once
#include <string>

#include "uccl_net.h"

namespace uccl {

// The built-in plugin ("Socket"): TCP, host pointers only, works on loopback.
ucclNet_t* builtinSocketPlugin();

// Validates `path` (non-empty, no ".." component, ends in ".so"), dlopens it RTLD_NOW|RTLD_LOCAL
// and returns its `ucclNetPlugin_v1` table.  On failure returns nullptr and fills `why`.
ucclNet_t* loadNetPlugin(const std::string& path, std::string* why);

// UCCL_NET_PLUGIN (cfgPath) if set and loadable, else the built-in socket plugin.
ucclNet_t* autoLoadNetPlugin(const std::string& cfgPath);

// Checks that every slot of the table is populated.
bool netPluginComplete(const ucclNet_t* net, std::string* why);

}  // namespace uccl
