// Collectives for communicators whose buffers live in host memory (the CPU backend), and the
// reduction / conversion helpers they share with the tests.
//
// The reference has no host implementation of its collectives; its only complete multi-rank data
// path is the network ring kernel that talks to the proxy through FIFOs and bounce slots
// (src/algorithms/ring.cc:170-279, src/device/primitives.hpp:223-341).  The CPU backend runs that
// same schedule with the calling thread in the kernel's role, so bootstrap, channels, FIFOs, the
// proxy thread and the network plugin are exercised without a GPU.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <vector>

#include "../core/comm.h"

namespace uccl {

// dst[i] += src[i] (fp32 accumulate for 16-bit types), count elements.
void hostReduceInto(void* dst, const void* src, size_t count, ucclDataType_t dt);
float bf16ToFloat(uint16_t v);
uint16_t floatToBf16(float f);
float halfToFloat(uint16_t v);
uint16_t floatToHalf(float f);

// One directed transfer of `len` bytes; sub-chunk j travels on conns[j % conns.size()].
struct HostXfer {
  std::vector<NetConn*> conns;
  bool isSend = false;
  const char* src = nullptr;  // send
  char* dst = nullptr;        // recv
  size_t len = 0;
  bool reduce = false;        // recv: dst += incoming instead of dst = incoming
  ucclDataType_t dtype = ucclUint8;
  // progress
  size_t posted = 0, done = 0;
  std::vector<uint64_t> steps;  // fifo step of each posted sub-chunk
};
// Runs all transfers to completion concurrently (single thread, no blocking on any one of them).
ucclResult_t hostRunXfers(Comm* comm, std::vector<HostXfer>& xfers);

ucclResult_t hostAllReduce(Comm* c, const void* send, void* recv, size_t count, ucclDataType_t dt);
ucclResult_t hostAllGather(Comm* c, const void* send, void* recv, size_t sendcount, ucclDataType_t dt);
ucclResult_t hostReduceScatter(Comm* c, const void* send, void* recv, size_t recvcount, ucclDataType_t dt);
ucclResult_t hostBroadcast(Comm* c, const void* send, void* recv, size_t count, ucclDataType_t dt, int root);
ucclResult_t hostReduce(Comm* c, const void* send, void* recv, size_t count, ucclDataType_t dt, int root);
ucclResult_t hostAllToAll(Comm* c, const void* send, void* recv, size_t count, ucclDataType_t dt);
struct HostP2pOp {
  bool isSend;
  int peer;
  const void* send;
  void* recv;
  size_t bytes;
};
ucclResult_t hostSendRecv(Comm* c, const std::vector<HostP2pOp>& ops);

}  // namespace uccl
