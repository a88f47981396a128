// Scheduler between the public entry points and the device / host algorithms: resolves buffers
// (symmetric or staged), asks the tuner for algorithm / protocol / CTA count and launches.
#pragma once
#include <cuda_runtime.h>

#include <vector>

#include "comm.h"

namespace uccl {

struct CollOp {
  ucclCollKind_t kind = ucclCollAllReduce;
  Comm* comm = nullptr;
  const void* send = nullptr;
  void* recv = nullptr;
  size_t count = 0;
  ucclDataType_t dtype = ucclBfloat16;
  int root = 0;        // broadcast / reduce root, or send/recv peer
  bool isSend = false; // point-to-point direction
  cudaStream_t stream = nullptr;
};

// Runs one collective now (called directly, or from ucclGroupEnd).
ucclResult_t executeOp(const CollOp& op);
// Runs a batch of point-to-point operations of one communicator as a single launch.
ucclResult_t executeP2pBatch(Comm* comm, const std::vector<CollOp>& ops);

// group.cc
bool groupActive();
ucclResult_t groupAppend(const CollOp& op);

// What the tuner decides for a call (exposed for ucclCommQueryTuning and the tests).
TuneChoice chooseFor(Comm* c, ucclCollKind_t kind, size_t bytes, bool symmetric, bool nvls, ucclDataType_t dt);

// Staging area inside the arena.
size_t stagingOffset(const Comm* c);

// device-side algorithms that live in their own translation units
ucclResult_t enqueueRing(Comm* c, const CollOp& op, ucclProto_t proto, int blocks);
ucclResult_t enqueueCopyEngine(Comm* c, const CollOp& op);
// A stream-ordered barrier among the ranks of the NVLink domain (one tiny kernel).
ucclResult_t enqueueBarrier(Comm* c, cudaStream_t s);
// device-to-device copy on a side stream, concurrent with what follows on `s` until sideCopyEnd
ucclResult_t sideCopyBegin(Comm* c, void* dst, const void* src, size_t bytes, cudaStream_t s);
ucclResult_t sideCopyEnd(Comm* c, cudaStream_t s);
// copy-engine all-gather with per-row-block arrival flags (all-gather -> GEMM fusion)
ucclResult_t allGatherPushBegin(Comm* c, const void* shard, char* const* fullPeer, char* const* readyPeer,
                                size_t shardBytes, int blocksPerRank, bool copyOwn, int lanes, cudaStream_t s);
ucclResult_t allGatherPushEnd(Comm* c, bool copyOwn, int lanes, cudaStream_t s);
ucclResult_t enqueueNetGpu(Comm* c, const CollOp& op);
ucclResult_t enqueueNetGpuP2p(Comm* c, const std::vector<CollOp>& ops);

}  // namespace uccl
