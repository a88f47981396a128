// One-sided windows (host side).
#pragma once
#include "../core/comm.h"

namespace uccl {
struct Window;
void rmaDestroyAll(Comm* c);
}  // namespace uccl
