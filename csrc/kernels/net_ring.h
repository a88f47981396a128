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
  size_t elemOff;       // this channel's slice, in elements: of the message (all-reduce, broadcast,
  size_t elemCount;     // reduce) or of every rank chunk (all-gather, reduce-scatter)
};

enum NetRingColl : int {
  NET_RING_ALLREDUCE = 0,      // buf holds the input; reduced in place
  NET_RING_ALLGATHER = 1,      // buf = [nranks][chunkElems], my chunk already in its place
  NET_RING_REDUCESCATTER = 2,  // buf = [nranks][chunkElems] work copy of the input; chunk `myRank` ends up reduced
  NET_RING_BROADCAST = 3,      // buf holds the message at the root and receives it elsewhere
  NET_RING_REDUCE = 4,         // buf holds the input (the root's copy receives the sum)
};

struct NetRingArgs {
  DevComm dc;
  char* buf;            // work buffer, see NetRingColl
  int dtype;
  int coll;             // NetRingColl
  int nranks, ringPos;  // size of the ring and my position in it
  int prevRank, nextRank;
  int rootPos;          // broadcast / reduce: ring position of the root
  int ringRanks[UCCL_MAX_RANKS];  // ring position -> rank (whose chunk sits at that index of buf)
  int nChannels;
  size_t slotBytes;
  size_t chunkElems;    // all-gather / reduce-scatter: elements per rank chunk
  NetRingChannel ch[UCCL_MAX_CHANNELS];
};

cudaError_t launchNetRingKernel(const NetRingArgs& a, cudaStream_t stream);

}  // namespace uccl
