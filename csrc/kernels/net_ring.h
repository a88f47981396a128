// Arguments of the GPU-driven network ring (see net_ring.cu).
#pragma once
#include <cuda_runtime.h>

#include "../transport/fifo.h"
#include "coll_device_types.h"
#include "device_comm.h"

namespace uccl {

struct NetRingChannel {
  ConnFifo* sendFifo;   // device aliases of mapped pinned host memory
  ConnFifo* recvFifo;
  char* sendBounce;
  char* recvBounce;
  size_t elemOff;       // this channel's slice of the message, in elements
  size_t elemCount;
};

struct NetRingArgs {
  DevComm dc;
  char* buf;            // work buffer (the receive buffer; already holds this rank's input)
  int dtype;
  int nranks, ringPos;  // size of the ring and my position in it
  int prevRank, nextRank;
  int nChannels;
  size_t slotBytes;
  NetRingChannel ch[UCCL_MAX_CHANNELS];
};

cudaError_t launchNetRingKernel(const NetRingArgs& a, cudaStream_t stream);

}  // namespace uccl
