// One directed network connection as the proxy thread and its producer see it: a FIFO, a set of
// bounce slots registered with the plugin, and the plugin's send or receive handle.
//
// The reference gives every channel a send FIFO + 8 bounce slots towards the ring successor and
// a receive FIFO + 8 slots from the predecessor (src/channel.cc:31-135, src/include/channel.h:16-67)
// and exchanges the listen addresses with MPI_Sendrecv (src/transport/net.cc:31-113).  The same
// object is used here for ring neighbours (connected at communicator creation through one
// bootstrap all-gather) and for arbitrary peers (connected on first use through tagged bootstrap
// messages), so send/recv and all-to-all can also run over the plugin.
#pragma once
#include <stdint.h>

#include <mutex>
#include <vector>

#include "fifo.h"
#include "uccl_net.h"

namespace uccl {

struct Comm;

struct NetConn {
  bool isSend = false;
  int peer = -1;
  int channel = 0;
  // shared with the producer
  ConnFifo* fifo = nullptr;     // host address
  ConnFifo* fifoDev = nullptr;  // device alias (mapped pinned memory) or == fifo on CPU
  char* bounce = nullptr;       // UCCL_STEPS slots of slotBytes each (host address)
  char* bounceDev = nullptr;    // device alias
  size_t slotBytes = 0;
  bool bounceOnDevice = false;  // plugin accepted UCCL_PTR_DEVICE registration
  // plugin side
  void* netComm = nullptr;
  void* listenComm = nullptr;
  void* mhandle[UCCL_STEPS] = {};
  // proxy-private
  uint64_t posted = 0;
  void* request[UCCL_STEPS] = {};
  // producer-private (CPU backend and host-driven paths)
  uint64_t step = 0;
};

// Allocation / teardown (pinned + mapped when the communicator is on a GPU).
ucclResult_t netConnAlloc(Comm* comm, NetConn* c, bool isSend, int peer, int channel);
void netConnFree(Comm* comm, NetConn* c);

// Ring neighbours of every channel; collective over the communicator.
ucclResult_t netSetupRings(Comm* comm);
// Connection to / from an arbitrary peer, created on first use.  The sender calls
// netGetSendConn(peer) while the receiver calls netGetRecvConn(sender).
ucclResult_t netEnsurePeers(Comm* comm, const std::vector<int>& peers);
ucclResult_t netGetSendConn(Comm* comm, int peer, NetConn** out);
ucclResult_t netGetRecvConn(Comm* comm, int peer, NetConn** out);
void netTeardown(Comm* comm);

// Producer-side helpers for host code (CPU backend): block until a slot is free / an operation
// completed, watching the abort word and the connection's error word.
// netHostAcquire: wait until the slot of the next step is reusable and return its address (a
// sender fills it before posting).  netHostPost: publish the next step.  netHostWait: wait for a
// posted step to complete.
ucclResult_t netHostAcquire(Comm* comm, NetConn* c, char** slot);
ucclResult_t netHostPost(Comm* comm, NetConn* c, uint32_t op, size_t bytes, uint64_t* stepOut);
ucclResult_t netHostWait(Comm* comm, NetConn* c, uint64_t step, size_t* bytesOut);
inline char* netSlot(NetConn* c, uint64_t step) { return c->bounce + (step % UCCL_STEPS) * c->slotBytes; }

}  // namespace uccl
