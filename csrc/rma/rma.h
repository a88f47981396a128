// One-sided windows (host side).
//
// The reference's window (src/rma/rma.h:37-50, src/rma/rma.cc:35-211) holds the local buffer, one
// IPC-mapped pointer per peer, a device array of 64-bit signal counters (slot p counts signals
// received from rank p) and IPC-mapped pointers to every peer's counter array.  Same content
// here; the mapping comes from the symmetric heap when the buffer was allocated with
// ucclMemAlloc, and from cudaIpc handles otherwise, and the counters live in the arena.
#pragma once
#include "../core/comm.h"
#include "uccl_device.cuh"

namespace uccl {

constexpr int kMaxWindows = 64;
constexpr size_t kArenaWinSignalOff = 160u << 10;  // u64 [kMaxWindows][UCCL_MAX_LOCAL_RANKS]

struct Window {
  uint32_t magic = 0x57494e44;
  Comm* comm = nullptr;
  int slot = -1;
  char* localBuff = nullptr;
  size_t size = 0;
  char* remotePtrs[UCCL_MAX_LOCAL_RANKS] = {};
  bool ipcOpened[UCCL_MAX_LOCAL_RANKS] = {};
  char* ipcBase[UCCL_MAX_LOCAL_RANKS] = {};
  uint64_t* localSignals = nullptr;
  uint64_t* remoteSignals[UCCL_MAX_LOCAL_RANKS] = {};
  void* dynTables = nullptr;  // device copy of remotePtrs | remoteSignals for ucclDeviceWindowDyn, made on demand
};

void rmaDestroyAll(Comm* c);

}  // namespace uccl
