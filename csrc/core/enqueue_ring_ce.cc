// Ring and copy-engine variants of all-reduce / all-gather / reduce-scatter.
//
// Ring: one persistent kernel, see kernels/ring.cu.
//
// Copy engine: the data movement is done by the GPUs' DMA engines (cudaMemcpyAsync peer copies
// on one side stream per peer) and only the summation runs on SMs, which leaves the SMs to the
// application -- the purpose of the reference's UCCL_EXEC_MODE=copy_engine
// (src/algorithms/copy_engine.cc:43-337, src/include/hw_resources.h:40-75).  Differences: copies
// are pull-only (the reference's all-gather pushes and pulls the same data,
// copy_engine.cc:160-226), nothing waits on the host (the reference calls event.wait() after each
// copy and queue.wait() at the end), and ranks meet in a device-side barrier before peers' memory
// is read and after it has been read (the reference notes the missing barrier at
// copy_engine.cc:88-97).
#include <string.h>

#include <stdlib.h>

#include <algorithm>

#include "../kernels/coll_device_types.h"
#include "../kernels/collectives.cuh"
#include "cuda_driver.h"
#include "enqueue.h"
#include "log.h"

namespace uccl {

namespace {

int devDtype(ucclDataType_t dt) {
  return dt == ucclFloat16 ? DEVDT_F16 : (dt == ucclBfloat16 ? DEVDT_BF16 : DEVDT_F32);
}

ucclResult_t cudaFail(Comm* c, const char* what) {
  commSetError(c, "%s: %s", what, cudaGetErrorString(cudaGetLastError()));
  return ucclSystemError;
}

ucclResult_t ensureCeStreams(Comm* c) {
  if (c->ceReady) return ucclSuccess;
  for (int p = 0; p < c->localRanks; ++p) {
    if (cudaStreamCreateWithFlags(&c->ceStream[p], cudaStreamNonBlocking) != cudaSuccess) return cudaFail(c, "cudaStreamCreate");
    if (cudaEventCreateWithFlags(&c->ceEvent[p], cudaEventDisableTiming) != cudaSuccess) return cudaFail(c, "cudaEventCreate");
  }
  if (cudaEventCreateWithFlags(&c->ceStart, cudaEventDisableTiming) != cudaSuccess) return cudaFail(c, "cudaEventCreate");
  c->ceReady = true;
  return ucclSuccess;
}

ucclResult_t barrierOnStream(Comm* c, cudaStream_t s) { return enqueueBarrier(c, s); }

// fan out: side streams wait for everything enqueued on `s` so far
ucclResult_t forkStreams(Comm* c, cudaStream_t s) {
  if (cudaEventRecord(c->ceStart, s) != cudaSuccess) return cudaFail(c, "cudaEventRecord");
  for (int p = 0; p < c->localRanks; ++p)
    if (cudaStreamWaitEvent(c->ceStream[p], c->ceStart, 0) != cudaSuccess) return cudaFail(c, "cudaStreamWaitEvent");
  return ucclSuccess;
}
// fan in: `s` waits for every side stream
ucclResult_t joinStreams(Comm* c, cudaStream_t s) {
  for (int p = 0; p < c->localRanks; ++p) {
    if (cudaEventRecord(c->ceEvent[p], c->ceStream[p]) != cudaSuccess) return cudaFail(c, "cudaEventRecord");
    if (cudaStreamWaitEvent(s, c->ceEvent[p], 0) != cudaSuccess) return cudaFail(c, "cudaStreamWaitEvent");
  }
  return ucclSuccess;
}

}  // namespace

// A device-to-device copy that runs on a side stream next to whatever follows on `s`:
// sideCopyBegin forks after the work already enqueued on `s`, sideCopyEnd makes `s` wait for it.
ucclResult_t sideCopyBegin(Comm* c, void* dst, const void* src, size_t bytes, cudaStream_t s) {
  const ucclResult_t r = ensureCeStreams(c);
  if (r != ucclSuccess) return r;
  if (cudaEventRecord(c->ceStart, s) != cudaSuccess) return cudaFail(c, "cudaEventRecord");
  if (cudaStreamWaitEvent(c->ceStream[0], c->ceStart, 0) != cudaSuccess) return cudaFail(c, "cudaStreamWaitEvent");
  if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, c->ceStream[0]) != cudaSuccess)
    return cudaFail(c, "cudaMemcpyAsync");
  return ucclSuccess;
}
// All-gather by copy engines for the all-gather -> GEMM fusion: this rank's shard goes to rows
// [rank * rows, ...) of every rank's A buffer in `chunks` pieces per peer, each followed (in stream
// order, on the same side stream) by a copy of ones onto the peer's arrival flags of the row
// blocks it covers (one contiguous copy: flags are 128 bytes apart and the source has zeros in
// between).  The GEMM kernel launched on `s` meanwhile polls those flags.
// lanes == 0: one side stream per peer, all peers at once.  lanes > 0: that many streams, and the
// peers are served in the order me-1, me-2, ... round-robin over the lanes, so that every rank
// receives its shards one after the other, nearest first (from me+1, me+2, ...) - the order in
// which the GEMM then visits them - instead of all of them at the very end.
// Call allGatherPushEnd after the kernel launch.
namespace {
// a column of 32-bit ones at the flag stride, the source of every copy-engine flag write
ucclResult_t ensureOnes(Comm* c) {
  if (c->onesDev) return ucclSuccess;
  if (cudaMalloc(&c->onesDev, kGemmFlagStrideBytes * kGemmMaxRowBlocks) != cudaSuccess) return cudaFail(c, "cudaMalloc");
  if (cudaMemset(c->onesDev, 0, kGemmFlagStrideBytes * kGemmMaxRowBlocks) != cudaSuccess ||
      cudaMemset2D(c->onesDev, kGemmFlagStrideBytes, 1, 1, kGemmMaxRowBlocks) != cudaSuccess)
    return cudaFail(c, "cudaMemset2D");
  return ucclSuccess;
}

int cePushStreams(Comm* c, int lanes, bool copyOwn, cudaStream_t* out) {
  const int n = c->localRanks, me = c->localRank;
  int k = 0;
  if (lanes <= 0) {
    for (int p = 0; p < n; ++p)
      if (p != me) out[k++] = c->ceStream[p];
    if (copyOwn) out[k++] = c->ceStream[me];
    return k;
  }
  const int used = std::min(lanes, n - 1);
  for (int i = 0; i < used; ++i) out[k++] = c->ceStream[i];
  if (copyOwn) out[k++] = c->ceStream[used];  // n streams exist and used <= n - 1
  return k;
}
}  // namespace

ucclResult_t allGatherPushBegin(Comm* c, const void* shard, char* const* fullPeer, char* const* readyPeer,
                                size_t shardBytes, int blocksPerRank, bool copyOwn, int lanes, cudaStream_t s) {
  const ucclResult_t r = ensureCeStreams(c);
  if (r != ucclSuccess) return r;
  const int n = c->localRanks, me = c->localRank;
  const ucclResult_t ro = ensureOnes(c);
  if (ro != ucclSuccess) return ro;
  cudaStream_t streams[UCCL_MAX_LOCAL_RANKS + 1];
  const int nstreams = cePushStreams(c, lanes, copyOwn, streams);
  if (cudaEventRecord(c->ceStart, s) != cudaSuccess) return cudaFail(c, "cudaEventRecord");
  for (int i = 0; i < nstreams; ++i)
    if (cudaStreamWaitEvent(streams[i], c->ceStart, 0) != cudaSuccess) return cudaFail(c, "cudaStreamWaitEvent");
  const size_t blkBytes = shardBytes / blocksPerRank;
  int wantChunks = c->fusedCeChunks > 0 ? c->fusedCeChunks : (c->cfg.fusedCeChunks > 0 ? c->cfg.fusedCeChunks : 2);
  if (const char* e = getenv("UCCL_FUSED_CE_CHUNKS")) {  // read per call so that a tuning run can vary it
    if (atoi(e) > 0) wantChunks = atoi(e);
  }
  const int chunks = std::min(wantChunks, blocksPerRank);
  const char* src = static_cast<const char*>(shard);
  const size_t rowOff = static_cast<size_t>(me) * shardBytes;
  const int usedLanes = lanes > 0 ? std::min(lanes, n - 1) : 0;
  auto pushChunk = [&](int p, int j, cudaStream_t st) -> ucclResult_t {
    const int b0 = static_cast<int>(static_cast<long long>(blocksPerRank) * j / chunks);
    const int b1 = static_cast<int>(static_cast<long long>(blocksPerRank) * (j + 1) / chunks);
    if (b1 == b0) return ucclSuccess;
    const size_t off = b0 * blkBytes, len = (b1 - b0) * blkBytes;
    if (cudaMemcpyAsync(fullPeer[p] + rowOff + off, src + off, len, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return cudaFail(c, "cudaMemcpyAsync");
    if (cudaMemcpyAsync(readyPeer[p] + (static_cast<size_t>(me) * blocksPerRank + b0) * kGemmFlagStrideBytes, c->onesDev,
                        static_cast<size_t>(b1 - b0) * kGemmFlagStrideBytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      return cudaFail(c, "cudaMemcpyAsync");
    return ucclSuccess;
  };
  if (usedLanes == 0) {
    for (int j = 0; j < chunks; ++j)
      for (int q = 1; q < n; ++q) {
        const int p = (me + q) % n;
        const ucclResult_t rr = pushChunk(p, j, c->ceStream[p]);
        if (rr != ucclSuccess) return rr;
      }
  } else {
    for (int q = 1; q < n; ++q) {
      const int p = (me - q + n) % n;  // rank p sees me at distance q
      for (int j = 0; j < chunks; ++j) {
        const ucclResult_t rr = pushChunk(p, j, c->ceStream[(q - 1) % usedLanes]);
        if (rr != ucclSuccess) return rr;
      }
    }
  }
  if (copyOwn && cudaMemcpyAsync(fullPeer[me] + rowOff, src, shardBytes, cudaMemcpyDeviceToDevice,
                                 streams[nstreams - 1]) != cudaSuccess)
    return cudaFail(c, "cudaMemcpyAsync");
  return ucclSuccess;
}
ucclResult_t allGatherPushEnd(Comm* c, bool copyOwn, int lanes, cudaStream_t s) {
  cudaStream_t streams[UCCL_MAX_LOCAL_RANKS + 1];
  const int nstreams = cePushStreams(c, lanes, copyOwn, streams);
  for (int i = 0; i < nstreams; ++i) {
    // one event per stream: the events array has an entry for every local rank
    if (cudaEventRecord(c->ceEvent[i], streams[i]) != cudaSuccess) return cudaFail(c, "cudaEventRecord");
    if (cudaStreamWaitEvent(s, c->ceEvent[i], 0) != cudaSuccess) return cudaFail(c, "cudaStreamWaitEvent");
  }
  return ucclSuccess;
}

ucclResult_t sideCopyEnd(Comm* c, cudaStream_t s) {
  if (cudaEventRecord(c->ceEvent[0], c->ceStream[0]) != cudaSuccess) return cudaFail(c, "cudaEventRecord");
  if (cudaStreamWaitEvent(s, c->ceEvent[0], 0) != cudaSuccess) return cudaFail(c, "cudaStreamWaitEvent");
  return ucclSuccess;
}

namespace {

ucclResult_t localReduce(Comm* c, char* dst, const char* slots, int nslots, size_t slotStride, size_t bytes,
                         ucclDataType_t dt, cudaStream_t s) {
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.dc = c->dev;
  a.dtype = devDtype(dt);
  a.in[0] = slots;
  a.out[0] = dst;
  a.inStride = slotStride;
  a.bytes = (bytes + 15) & ~size_t(15);
  a.userBytes = bytes;
  a.root = nslots;
  int blocks = static_cast<int>(std::min<size_t>(32, std::max<size_t>(1, bytes / (256u << 10))));
  if (launchCollKernel(KERN_LOCAL_REDUCE, a, blocks, s) != cudaSuccess) return cudaFail(c, "reduce kernel launch");
  return ucclSuccess;
}

#define UCCL_TRY(x)                   \
  do {                                \
    ucclResult_t _r = (x);            \
    if (_r != ucclSuccess) return _r; \
  } while (0)

}  // namespace

ucclResult_t enqueueBarrier(Comm* c, cudaStream_t s) {
  CollArgs a;
  memset(&a, 0, sizeof(a));
  a.dc = c->dev;
  if (launchCollKernel(KERN_BARRIER, a, 1, s) != cudaSuccess) return cudaFail(c, "barrier kernel launch");
  return ucclSuccess;
}

ucclResult_t enqueueRing(Comm* c, const CollOp& op, ucclProto_t proto, int blocks) {
  const int n = c->localRanks;
  RingArgs a;
  memset(&a, 0, sizeof(a));
  a.dc = c->dev;
  a.inUser = static_cast<const char*>(op.send);
  a.outUser = static_cast<char*>(op.recv);
  a.count = op.count;
  a.dtype = devDtype(op.dtype);
  a.coll = op.kind;
  a.proto = proto;
  const Channel& ch = c->channels[0];
  a.ringPos = ch.index;
  for (int p = 0; p < n; ++p) {
    const int globalRank = ch.userRanks[((p - ch.index) % n + n) % n];
    a.ringRanks[p] = c->peers[globalRank].localRank;
  }
  a.ringNext = c->peers[ch.next].localRank;
  a.ringPrev = c->peers[ch.prev].localRank;
  a.ringBufOff = stagingOffset(c);
  a.ringBufBytes = c->cfg.stagingBytes & ~size_t(4095);
  const size_t es = dataTypeSize(op.dtype);
  if (proto == ucclProtoLL128) {
    blocks = std::min(blocks, kLLBlocks);
  } else {
    // every channel needs slots of at least one vector
    const int maxByBuf = static_cast<int>(a.ringBufBytes / (kRingSlots * 4096));
    blocks = std::min(blocks, std::max(1, maxByBuf));
  }
  // no more channels than elements per chunk
  const size_t perChunk = op.kind == ucclCollAllReduce ? op.count / static_cast<size_t>(n) : op.count;
  const size_t minPerChan = std::max<size_t>(1, 4096 / es);
  blocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(blocks, (perChunk + minPerChan - 1) / minPerChan)));
  if (c->cfg.maxCtas > 0) blocks = std::min(blocks, c->cfg.maxCtas);
  cudaError_t e = launchRingKernel(a, blocks, op.stream);
  if (e != cudaSuccess) {
    commSetError(c, "ring kernel launch failed: %s", cudaGetErrorString(e));
    return ucclSystemError;
  }
  return ucclSuccess;
}

ucclResult_t enqueueCopyEngine(Comm* c, const CollOp& op) {
  UCCL_TRY(ensureCeStreams(c));
  const int n = c->localRanks, me = c->localRank;
  const size_t es = dataTypeSize(op.dtype);
  cudaStream_t s = op.stream;
  const size_t stageOff = stagingOffset(c);
  const size_t stageBytes = c->cfg.stagingBytes & ~size_t(4095);
  char* stagePeer[UCCL_MAX_LOCAL_RANKS];
  for (int p = 0; p < n; ++p) stagePeer[p] = c->arena->peer[p] + stageOff;
  char* stage = stagePeer[me];
  const char* send = static_cast<const char*>(op.send);
  char* recv = static_cast<char*>(op.recv);
  auto copy = [&](void* dst, const void* src, size_t bytes, cudaStream_t st) -> ucclResult_t {
    if (bytes == 0 || dst == src) return ucclSuccess;  // in place: my own part is already where it belongs
    if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return cudaFail(c, "cudaMemcpyAsync");
    return ucclSuccess;
  };

  if (op.kind == ucclCollAllGather) {
    const size_t chunk = op.count * es;
    const size_t cap = stageBytes;
    for (size_t po = 0; po < chunk; po += cap) {
      const size_t len = std::min(cap, chunk - po);
      UCCL_TRY(copy(stage, send + po, len, s));                    // expose my piece
      UCCL_TRY(barrierOnStream(c, s));
      UCCL_TRY(forkStreams(c, s));
      for (int k = 0; k < n; ++k) {
        const int p = (me + k) % n;
        UCCL_TRY(copy(recv + static_cast<size_t>(p) * chunk + po, p == me ? send + po : stagePeer[p], len, c->ceStream[p]));
      }
      UCCL_TRY(joinStreams(c, s));
      UCCL_TRY(barrierOnStream(c, s));                             // peers finished reading my piece
    }
    return ucclSuccess;
  }

  if (op.kind == ucclCollReduceScatter) {
    const size_t chunk = op.count * es;
    // staging: [0, half) my input pieces for all n chunks, [half, 2*half) pulled slots
    const size_t half = (stageBytes / 2) & ~size_t(255);
    const size_t cap = (half / n) & ~size_t(15);
    for (size_t po = 0; po < chunk; po += cap) {
      const size_t len = std::min(cap, chunk - po);
      for (int q = 0; q < n; ++q)
        UCCL_TRY(copy(stage + static_cast<size_t>(q) * cap, send + static_cast<size_t>(q) * chunk + po, len, s));
      UCCL_TRY(barrierOnStream(c, s));
      UCCL_TRY(forkStreams(c, s));
      for (int k = 0; k < n; ++k) {
        const int p = (me + k) % n;
        UCCL_TRY(copy(stage + half + static_cast<size_t>(p) * cap, stagePeer[p] + static_cast<size_t>(me) * cap, len, c->ceStream[p]));
      }
      UCCL_TRY(joinStreams(c, s));
      UCCL_TRY(localReduce(c, recv + po, stage + half, n, cap, len, op.dtype, s));
      UCCL_TRY(barrierOnStream(c, s));
    }
    return ucclSuccess;
  }

  // all-reduce = reduce-scatter into a staged shard, then all-gather of the shards
  const size_t bytes = op.count * es;
  // staging thirds: input copy | pulled slots | reduced shard
  const size_t third = (stageBytes / 3) & ~size_t(255);
  const size_t capShard = (third / n) & ~size_t(15);
  const size_t cap = capShard * n;
  for (size_t po = 0; po < bytes; po += cap) {
    const size_t len = std::min(cap, bytes - po);
    // shard size in bytes: multiple of the element size, last shard takes what is left
    size_t shard = (len / n / es) * es;
    if (shard == 0) shard = es;
    auto shardOff = [&](int r) { return std::min(len, static_cast<size_t>(r) * shard); };
    auto shardLen = [&](int r) { return r == n - 1 ? len - shardOff(r) : std::min(shard, len - shardOff(r)); };
    UCCL_TRY(copy(stage, send + po, len, s));
    UCCL_TRY(barrierOnStream(c, s));
    UCCL_TRY(forkStreams(c, s));
    const size_t slotStride = ((shardLen(n - 1) > shard ? shardLen(n - 1) : shard) + 15) & ~size_t(15);
    for (int k = 0; k < n; ++k) {
      const int p = (me + k) % n;
      UCCL_TRY(copy(stage + third + static_cast<size_t>(p) * slotStride, stagePeer[p] + shardOff(me), shardLen(me), c->ceStream[p]));
    }
    UCCL_TRY(joinStreams(c, s));
    UCCL_TRY(localReduce(c, stage + 2 * third, stage + third, n, slotStride, shardLen(me), op.dtype, s));
    UCCL_TRY(barrierOnStream(c, s));  // every shard is reduced
    UCCL_TRY(forkStreams(c, s));
    for (int k = 0; k < n; ++k) {
      const int p = (me + k) % n;
      UCCL_TRY(copy(recv + po + shardOff(p), stagePeer[p] + 2 * third, shardLen(p), c->ceStream[p]));
    }
    UCCL_TRY(joinStreams(c, s));
    UCCL_TRY(barrierOnStream(c, s));  // peers finished reading my shard
  }
  return ucclSuccess;
}

}  // namespace uccl
