// Enqueue: algorithm selection and kernel launches for communicators on GPUs, dispatch to the
// host ring for communicators on CPUs.
//
// Counterpart of the reference's src/enqueue.cc:121-570.  Differences that matter:
//  * the single-rank case is a stream-ordered cudaMemcpyAsync (the reference blocks the host
//    with .wait(), src/enqueue.cc:208-213);
//  * a message is not cut into one launch per channel: one persistent kernel gets `blocks` CTAs;
//  * user buffers that came from ucclMemAlloc are used in place (zero copy, NVLS-capable);
//    any other buffer is staged through the arena inside the same kernel, in pieces if large;
//  * all-gather and reduce-scatter use all CTAs too (the reference confines them to channel 0,
//    src/enqueue.cc:431,544).
#include "enqueue.h"

#include <string.h>

#include <algorithm>

#include "../host/host_coll.h"
#include "../kernels/coll_device_types.h"
#include "../kernels/collectives.cuh"
#include "log.h"
#include "trace.h"

namespace uccl {

size_t stagingOffset(const Comm* c) {
  return kArenaP2pDataOff + static_cast<size_t>(c->localRanks) * kP2pSlots * kP2pSlotBytes;
}

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline size_t up16(size_t v) { return (v + 15) & ~size_t(15); }

int devDtype(ucclDataType_t dt) {
  switch (dt) {
    case ucclFloat16: return DEVDT_F16;
    case ucclBfloat16: return DEVDT_BF16;
    case ucclFloat32: return DEVDT_F32;
    default: return DEVDT_F32;  // copy-only kernels ignore it
  }
}
bool reducible(ucclDataType_t dt) { return dt == ucclFloat16 || dt == ucclBfloat16 || dt == ucclFloat32; }

// A user buffer that lies in a symmetric segment at a 16-byte aligned address.
struct SymRef {
  SymSegment* seg = nullptr;
  size_t off = 0;
  explicit operator bool() const { return seg != nullptr; }
};
SymRef symResolve(Comm* c, const void* p, size_t bytes) {
  SymRef r;
  if (!p || !aligned16(p)) return r;
  SymSegment* s = c->heap.find(p, bytes ? bytes : 1);
  if (!s) return r;
  r.seg = s;
  r.off = static_cast<size_t>(static_cast<const char*>(p) - s->local);
  return r;
}

struct Stage {
  char* peer[UCCL_MAX_LOCAL_RANKS];
  char* mc;
  size_t bytes;
};
Stage stageOf(Comm* c) {
  Stage s;
  const size_t off = stagingOffset(c);
  for (int i = 0; i < UCCL_MAX_LOCAL_RANKS; ++i) s.peer[i] = i < c->localRanks ? c->arena->peer[i] + off : nullptr;
  s.mc = c->arena->mc ? c->arena->mc + off : nullptr;
  s.bytes = c->cfg.stagingBytes & ~size_t(4095);
  return s;
}

void baseArgs(Comm* c, CollArgs* a, ucclDataType_t dt) {
  memset(a, 0, sizeof(*a));
  a->dc = c->dev;
  a->dtype = devDtype(dt);
}

ucclResult_t launch(Comm* c, CollKernel k, const CollArgs& a, int blocks, cudaStream_t s) {
  cudaError_t e = launchCollKernel(k, a, blocks, s);
  if (e != cudaSuccess) {
    commSetError(c, "kernel launch failed: %s", cudaGetErrorString(e));
    return ucclSystemError;
  }
  return ucclSuccess;
}

int capBlocks(Comm* c, int blocks) {
  int cap = c->cfg.maxCtas > 0 ? std::min(c->cfg.maxCtas, kMaxBlocks) : kMaxBlocks;
  return std::max(1, std::min(blocks, cap));
}

// ------------------------------------------------------------------ all-reduce
ucclResult_t arLL(Comm* c, const CollOp& op, size_t bytes) {
  CollArgs a;
  baseArgs(c, &a, op.dtype);
  a.inUser = static_cast<const char*>(op.send);
  a.outUser = static_cast<char*>(op.recv);
  a.bytes = a.userBytes = bytes;
  const int blocks = static_cast<int>((bytes + kLLDataPerBlock - 1) / kLLDataPerBlock);
  return launch(c, KERN_AR_LL, a, blocks, op.stream);
}

// all-gather / reduce-scatter as low-latency packets straight between the user buffers (see chunk_ll)
ucclResult_t chunkLL(Comm* c, const CollOp& op, size_t chunk, CollKernel kern) {
  CollArgs a;
  baseArgs(c, &a, kern == KERN_RS_LL ? op.dtype : ucclFloat32);  // gather and all-to-all move bytes, whatever the element type
  a.inUser = static_cast<const char*>(op.send);
  a.outUser = static_cast<char*>(op.recv);
  a.bytes = a.userBytes = chunk;
  a.inStride = a.outStride = chunk;
  const int blocks = std::max(1, static_cast<int>((chunk + kLLDataPerBlock - 1) / kLLDataPerBlock));
  return launch(c, kern, a, blocks, op.stream);
}

ucclResult_t arDirect(Comm* c, const CollOp& op, size_t bytes, const TuneChoice& ch) {
  const bool whole = (bytes & 15) == 0;
  SymRef sIn = whole ? symResolve(c, op.send, bytes) : SymRef();
  SymRef sOut = whole ? symResolve(c, op.recv, bytes) : SymRef();
  Stage st = stageOf(c);
  const int n = c->localRanks;
  const char* send = static_cast<const char*>(op.send);
  char* recv = static_cast<char*>(op.recv);

  ucclAlgo_t algo = ch.algo;
  if (algo == ucclAlgoNvls) {
    const bool inMc = sIn ? sIn.seg->mc != nullptr : st.mc != nullptr;
    const bool outMc = sOut ? sOut.seg->mc != nullptr : st.mc != nullptr;
    if (!inMc || !outMc) algo = ucclAlgoTwoShot;
  }
  const CollKernel kern = algo == ucclAlgoOneShot ? KERN_AR_ONESHOT : (algo == ucclAlgoNvls ? KERN_AR_NVLS : KERN_AR_TWOSHOT);

  if (algo == ucclAlgoOneShot) {
    // inputs must be peer-visible; the output is written locally only.  In place on a symmetric
    // buffer the output would overwrite what peers are still reading, so it takes a detour
    // through the staging area and is copied out after the closing barrier.
    const bool inPlaceSym = sIn && send == recv;
    const size_t cap = (sIn && !inPlaceSym) ? bytes : ((st.bytes / 2) & ~size_t(15));
    for (size_t po = 0; po < bytes; po += cap) {
      const size_t ub = std::min(cap, bytes - po), wb = up16(ub);
      CollArgs a;
      baseArgs(c, &a, op.dtype);
      a.bytes = wb;
      a.userBytes = ub;
      if (sIn) {
        for (int p = 0; p < n; ++p) a.in[p] = sIn.seg->peer[p] + sIn.off + po;
      } else {
        for (int p = 0; p < n; ++p) a.in[p] = st.peer[p];
        a.inUser = send + po;
      }
      if ((ub & 15) == 0 && !inPlaceSym) {
        a.out[c->localRank] = recv + po;
      } else {
        a.out[c->localRank] = st.peer[c->localRank] + st.bytes / 2;
        a.outUser = recv + po;
      }
      ucclResult_t r = launch(c, kern, a, capBlocks(c, ch.blocks), op.stream);
      if (r != ucclSuccess) return r;
    }
    return ucclSuccess;
  }

  // two-shot / NVLS: inputs and outputs must both be peer-visible
  const bool zeroCopy = sIn && sOut;
  const size_t cap = zeroCopy ? bytes : (st.bytes & ~size_t(255));
  for (size_t po = 0; po < bytes; po += cap) {
    const size_t ub = std::min(cap, bytes - po), wb = up16(ub);
    CollArgs a;
    baseArgs(c, &a, op.dtype);
    a.bytes = wb;
    a.userBytes = ub;
    if (zeroCopy) {
      for (int p = 0; p < n; ++p) {
        a.in[p] = sIn.seg->peer[p] + sIn.off + po;
        a.out[p] = sOut.seg->peer[p] + sOut.off + po;
      }
      a.inMc = sIn.seg->mc ? sIn.seg->mc + sIn.off + po : nullptr;
      a.outMc = sOut.seg->mc ? sOut.seg->mc + sOut.off + po : nullptr;
    } else {
      // staged, in place inside the staging area
      for (int p = 0; p < n; ++p) {
        a.in[p] = st.peer[p];
        a.out[p] = st.peer[p];
      }
      a.inMc = st.mc;
      a.outMc = st.mc;
      a.inUser = send + po;
      a.outUser = recv + po;
    }
    ucclResult_t r = launch(c, kern, a, capBlocks(c, ch.blocks), op.stream);
    if (r != ucclSuccess) return r;
  }
  return ucclSuccess;
}

// ------------------------------------------------------------------ all-gather
ucclResult_t agDirect(Comm* c, const CollOp& op, size_t chunk, const TuneChoice& ch) {
  const int n = c->localRanks;
  Stage st = stageOf(c);
  const char* send = static_cast<const char*>(op.send);
  char* recv = static_cast<char*>(op.recv);
  SymRef sOut = (chunk & 15) == 0 ? symResolve(c, recv, chunk * n) : SymRef();
  const int blocks = capBlocks(c, ch.blocks);
  if (sOut) {
    // every rank must take this branch together, so a misaligned source is first copied into
    // this rank's own slot of the (aligned, symmetric) output and pushed from there
    if (!aligned16(send)) {
      char* slot = recv + static_cast<size_t>(c->localRank) * chunk;
      if (cudaMemcpyAsync(slot, send, chunk, cudaMemcpyDeviceToDevice, op.stream) != cudaSuccess) return ucclSystemError;
      send = slot;
    }
    CollArgs a;
    baseArgs(c, &a, op.dtype);
    a.inUser = send;
    for (int p = 0; p < n; ++p) a.out[p] = sOut.seg->peer[p] + sOut.off;
    a.outMc = (ch.algo == ucclAlgoNvls && sOut.seg->mc) ? sOut.seg->mc + sOut.off : nullptr;
    a.chunkBytes = a.userBytes = chunk;
    a.outStride = chunk;
    return launch(c, KERN_AG_PUSH, a, blocks, op.stream);
  }
  SymRef sIn = symResolve(c, send, chunk);
  const size_t cap = sIn ? chunk : (st.bytes & ~size_t(15));
  for (size_t po = 0; po < chunk; po += cap) {
    const size_t len = std::min(cap, chunk - po);
    CollArgs a;
    baseArgs(c, &a, op.dtype);
    if (sIn) {
      for (int p = 0; p < n; ++p) a.in[p] = sIn.seg->peer[p] + sIn.off + po;
    } else {
      for (int p = 0; p < n; ++p) a.in[p] = st.peer[p];
      a.inUser = send + po;
    }
    a.outUser = recv + po;
    a.outStride = chunk;
    a.chunkBytes = a.userBytes = len;
    ucclResult_t r = launch(c, KERN_AG_PULL, a, blocks, op.stream);
    if (r != ucclSuccess) return r;
  }
  return ucclSuccess;
}

// ------------------------------------------------------------------ reduce-scatter
ucclResult_t rsDirect(Comm* c, const CollOp& op, size_t chunk, const TuneChoice& ch) {
  const int n = c->localRanks;
  Stage st = stageOf(c);
  const char* send = static_cast<const char*>(op.send);
  char* recv = static_cast<char*>(op.recv);
  const int blocks = capBlocks(c, ch.blocks);
  SymRef sIn = (chunk & 15) == 0 ? symResolve(c, send, chunk * n) : SymRef();
  if (sIn) {
    CollArgs a;
    baseArgs(c, &a, op.dtype);
    for (int p = 0; p < n; ++p) a.in[p] = sIn.seg->peer[p] + sIn.off;
    a.inMc = (ch.algo == ucclAlgoNvls && sIn.seg->mc) ? sIn.seg->mc + sIn.off : nullptr;
    a.inStride = chunk;
    a.chunkBytes = a.userBytes = chunk;
    a.out[c->localRank] = recv;  // any alignment: the kernel narrows its stores if needed
    return launch(c, KERN_RS_PULL, a, blocks, op.stream);
  }
  // staged: the first half of the staging area holds n padded pieces, the second half results
  const size_t half = (st.bytes / 2) & ~size_t(15);
  const size_t cap = (half / n) & ~size_t(15);
  for (size_t po = 0; po < chunk; po += cap) {
    const size_t len = std::min(cap, chunk - po), padded = up16(len);
    CollArgs a;
    baseArgs(c, &a, op.dtype);
    for (int p = 0; p < n; ++p) a.in[p] = st.peer[p];
    a.inMc = (ch.algo == ucclAlgoNvls && st.mc) ? st.mc : nullptr;
    a.inUser = send + po;
    a.inStride = chunk;
    a.chunkBytes = padded;
    a.userBytes = len;
    if ((len & 15) == 0) {
      a.out[c->localRank] = recv + po;
    } else {
      a.out[c->localRank] = st.peer[c->localRank] + half;
      a.outUser = recv + po;
    }
    ucclResult_t r = launch(c, KERN_RS_PULL, a, blocks, op.stream);
    if (r != ucclSuccess) return r;
  }
  return ucclSuccess;
}

// ------------------------------------------------------------------ broadcast
ucclResult_t bcastDirect(Comm* c, const CollOp& op, size_t bytes, const TuneChoice& ch) {
  const int n = c->localRanks;
  Stage st = stageOf(c);
  const char* send = static_cast<const char*>(op.send);
  char* recv = static_cast<char*>(op.recv);
  const int blocks = capBlocks(c, ch.blocks);
  const int root = c->peers[op.root].localRank;
  SymRef sOut = (bytes & 15) == 0 ? symResolve(c, recv, bytes) : SymRef();
  if (sOut) {
    // the root pushes into everybody's (symmetric) receive buffer
    const char* src = send;
    if (c->localRank == root && !aligned16(send)) {
      if (cudaMemcpyAsync(recv, send, bytes, cudaMemcpyDeviceToDevice, op.stream) != cudaSuccess) return ucclSystemError;
      src = recv;
    }
    CollArgs a;
    baseArgs(c, &a, op.dtype);
    a.root = root;
    a.inUser = src;
    for (int p = 0; p < n; ++p) a.out[p] = sOut.seg->peer[p] + sOut.off;
    a.outMc = (ch.algo == ucclAlgoNvls && sOut.seg->mc) ? sOut.seg->mc + sOut.off : nullptr;
    a.bytes = a.userBytes = bytes;
    return launch(c, KERN_BCAST_PUSH, a, blocks, op.stream);
  }
  const size_t cap = st.bytes & ~size_t(15);
  for (size_t po = 0; po < bytes || po == 0; po += cap) {
    const size_t len = std::min(cap, bytes - po);
    CollArgs a;
    baseArgs(c, &a, op.dtype);
    a.root = root;
    for (int p = 0; p < n; ++p) a.in[p] = st.peer[p];
    a.inUser = c->localRank == root ? send + po : nullptr;
    a.outUser = recv + po;
    a.bytes = up16(len);
    a.userBytes = len;
    ucclResult_t r = launch(c, KERN_BCAST_PULL, a, blocks, op.stream);
    if (r != ucclSuccess) return r;
    if (bytes == 0) break;
  }
  return ucclSuccess;
}

// ------------------------------------------------------------------ reduce
ucclResult_t reduceDirect(Comm* c, const CollOp& op, size_t bytes, const TuneChoice& ch) {
  const int n = c->localRanks;
  Stage st = stageOf(c);
  const char* send = static_cast<const char*>(op.send);
  char* recv = static_cast<char*>(op.recv);
  const int blocks = capBlocks(c, ch.blocks);
  const int root = c->peers[op.root].localRank;
  const bool isRoot = c->localRank == root;
  SymRef sIn = (bytes & 15) == 0 ? symResolve(c, send, bytes) : SymRef();
  const size_t half = (st.bytes / 2) & ~size_t(15);
  const size_t cap = sIn ? bytes : half;
  for (size_t po = 0; po < bytes; po += cap) {
    const size_t len = std::min(cap, bytes - po);
    CollArgs a;
    baseArgs(c, &a, op.dtype);
    a.root = root;
    a.bytes = up16(len);
    a.userBytes = len;
    if (sIn) {
      for (int p = 0; p < n; ++p) a.in[p] = sIn.seg->peer[p] + sIn.off + po;
      a.inMc = (ch.algo == ucclAlgoNvls && sIn.seg->mc) ? sIn.seg->mc + sIn.off + po : nullptr;
    } else {
      for (int p = 0; p < n; ++p) a.in[p] = st.peer[p];
      a.inMc = (ch.algo == ucclAlgoNvls && st.mc) ? st.mc : nullptr;
      a.inUser = send + po;
    }
    if (isRoot) {
      if ((len & 15) == 0) {
        a.out[c->localRank] = recv + po;
      } else {
        a.out[c->localRank] = st.peer[c->localRank] + half;
        a.outUser = recv + po;
      }
    }
    ucclResult_t r = launch(c, KERN_REDUCE_PULL, a, blocks, op.stream);
    if (r != ucclSuccess) return r;
  }
  return ucclSuccess;
}

// ------------------------------------------------------------------ all-to-all
ucclResult_t a2aDirect(Comm* c, const CollOp& op, size_t chunk, const TuneChoice& ch) {
  const int n = c->localRanks;
  Stage st = stageOf(c);
  const char* send = static_cast<const char*>(op.send);
  char* recv = static_cast<char*>(op.recv);
  const int blocks = capBlocks(c, ch.blocks);
  SymRef sIn = symResolve(c, send, chunk * n);
  const size_t cap = sIn ? chunk : ((st.bytes / n) & ~size_t(15));
  for (size_t po = 0; po < chunk; po += cap) {
    const size_t len = std::min(cap, chunk - po);
    CollArgs a;
    baseArgs(c, &a, op.dtype);
    if (sIn) {
      for (int p = 0; p < n; ++p) a.in[p] = sIn.seg->peer[p] + sIn.off + po;
    } else {
      for (int p = 0; p < n; ++p) a.in[p] = st.peer[p];
      a.inUser = send + po;
    }
    a.inStride = chunk;
    a.outUser = recv + po;
    a.outStride = chunk;
    a.chunkBytes = a.userBytes = len;
    ucclResult_t r = launch(c, KERN_A2A_PULL, a, blocks, op.stream);
    if (r != ucclSuccess) return r;
  }
  return ucclSuccess;
}

ucclResult_t localCopy(Comm* c, const void* src, void* dst, size_t bytes, cudaStream_t s) {
  if (src == dst || bytes == 0) return ucclSuccess;
  if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s) != cudaSuccess) {
    commSetError(c, "cudaMemcpyAsync failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  return ucclSuccess;
}

ucclResult_t executeHost(const CollOp& op) {
  Comm* c = op.comm;
  switch (op.kind) {
    case ucclCollAllReduce: return hostAllReduce(c, op.send, op.recv, op.count, op.dtype);
    case ucclCollAllGather: return hostAllGather(c, op.send, op.recv, op.count, op.dtype);
    case ucclCollReduceScatter: return hostReduceScatter(c, op.send, op.recv, op.count, op.dtype);
    case ucclCollBroadcast: return hostBroadcast(c, op.send, op.recv, op.count, op.dtype, op.root);
    case ucclCollReduce: return hostReduce(c, op.send, op.recv, op.count, op.dtype, op.root);
    case ucclCollAllToAll: return hostAllToAll(c, op.send, op.recv, op.count, op.dtype);
    case ucclCollSendRecv: {
      std::vector<HostP2pOp> v(1);
      v[0] = {op.isSend, op.root, op.send, op.recv, op.count * dataTypeSize(op.dtype)};
      return hostSendRecv(c, v);
    }
    default: return ucclInternalError;
  }
}

}  // namespace

TuneChoice chooseFor(Comm* c, ucclCollKind_t kind, size_t bytes, bool symmetric, bool nvls, ucclDataType_t dt) {
  TuneQuery q;
  q.coll = kind;
  q.bytes = bytes;
  q.nranks = c->nRanks;
  q.nvls = nvls;
  q.symmetric = symmetric;
  q.reducible = reducible(dt);
  q.netOnly = c->useNet || !c->p2pReady;
  // copy_engine: copy engines move every byte (a small kernel reduces where the collective reduces);
  // hybrid: the same from 1 MiB up, SM kernels below, where the engines' start-up cost dominates
  q.copyEngine = c->cfg.execMode == EXEC_COPY_ENGINE || (c->cfg.execMode == EXEC_HYBRID && bytes >= (1u << 20));
  q.forcedAlgo = c->forcedAlgo;
  q.forcedProto = c->forcedProto;
  q.maxBlocks = c->cfg.maxCtas;
  TuneChoice ch = c->tuner.choose(q);
  if (c->forcedBlocks > 0) {
    int cap = (ch.proto == ucclProtoLL || ch.proto == ucclProtoLL128) ? kLLBlocks : kMaxBlocks;
    ch.blocks = std::min(c->forcedBlocks, cap);
  }
  return ch;
}

ucclResult_t executeOp(const CollOp& op) {
  Comm* c = op.comm;
  const size_t es = dataTypeSize(op.dtype);
  const int n = c->nRanks;
  size_t msgBytes = op.count * es;
  if (op.kind == ucclCollAllGather || op.kind == ucclCollReduceScatter || op.kind == ucclCollAllToAll)
    msgBytes *= static_cast<size_t>(n);

  if (c->backend == BACKEND_CPU) {
    commCount(c, op.kind, msgBytes, c->nRanks > 1 ? ucclAlgoNet : ucclAlgoAuto);
    return executeHost(op);
  }

  int prevDev = -1;
  cudaGetDevice(&prevDev);
  if (prevDev != c->cudaDev) cudaSetDevice(c->cudaDev);
  struct Restore {
    int d, cur;
    ~Restore() { if (d >= 0 && d != cur) cudaSetDevice(d); }
  } restore{prevDev, c->cudaDev};

  // a failure recorded by an earlier kernel is reported now
  if (c->hostFlags && __atomic_load_n(&c->hostFlags[8], __ATOMIC_ACQUIRE) != DEV_OK) {
    commPollDeviceStatus(c);
    return ucclRemoteError;
  }

  if (n == 1) {
    commCount(c, op.kind, msgBytes, ucclAlgoAuto);
    if (op.kind == ucclCollSendRecv) {
      commSetError(c, "send/recv to self needs a matching pair inside one group");
      return ucclInvalidUsage;
    }
    return localCopy(c, op.send, op.recv, op.count * es, op.stream);
  }

  TraceScope trace(c, collName(op.kind), msgBytes, op.stream);
  if (c->useNet || !c->p2pReady) {
    commCount(c, op.kind, msgBytes, ucclAlgoNet);
    trace.setAlgo(ucclAlgoNet);
    return enqueueNetGpu(c, op);
  }

  const size_t chunk = op.count * es;
  bool nvls = c->arena && c->arena->mc != nullptr;
  bool sym = false;
  if (op.kind != ucclCollSendRecv) {
    SymRef a = symResolve(c, op.send, 1), b = symResolve(c, op.recv, 1);
    sym = a || b;
  }
  TuneChoice ch = chooseFor(c, op.kind, msgBytes, sym, nvls, op.dtype);
  commCount(c, op.kind, msgBytes, ch.algo);
  trace.setAlgo(ch.algo);
  UCCL_LOG(TRACE, "%s bytes=%zu algo=%s proto=%s blocks=%d sym=%d", collName(op.kind), msgBytes, algoName(ch.algo),
           protoName(ch.proto), ch.blocks, (int)sym);

  if (ch.algo == ucclAlgoCopyEngine &&
      (op.kind == ucclCollAllReduce || op.kind == ucclCollAllGather || op.kind == ucclCollReduceScatter))
    return enqueueCopyEngine(c, op);
  if (ch.algo == ucclAlgoRing &&
      (op.kind == ucclCollAllReduce || op.kind == ucclCollAllGather || op.kind == ucclCollReduceScatter)) {
    if (reducible(op.dtype)) return enqueueRing(c, op, ch.proto == ucclProtoLL128 ? ucclProtoLL128 : ucclProtoSimple, ch.blocks);
    // copy-only element types (fp8, raw bytes) ride the ring as 4- or 2-byte words; an odd byte
    // count takes the direct kernels below
    if (op.kind == ucclCollAllGather && (chunk % 2) == 0) {
      CollOp w = op;
      w.dtype = (chunk % 4) == 0 ? ucclFloat32 : ucclFloat16;
      w.count = chunk / dataTypeSize(w.dtype);
      return enqueueRing(c, w, ch.proto == ucclProtoLL128 ? ucclProtoLL128 : ucclProtoSimple, ch.blocks);
    }
  }

  switch (op.kind) {
    case ucclCollAllReduce:
      if ((ch.proto == ucclProtoLL || ch.proto == ucclProtoLL128) &&
          chunk <= static_cast<size_t>(kLLBlocks) * kLLDataPerBlock)
        return arLL(c, op, chunk);
      return arDirect(c, op, chunk, ch);
    case ucclCollAllGather:
      if (ch.proto == ucclProtoLL && chunk <= static_cast<size_t>(kLLBlocks) * kLLDataPerBlock) return chunkLL(c, op, chunk, KERN_AG_LL);
      return agDirect(c, op, chunk, ch);
    case ucclCollReduceScatter:
      if (ch.proto == ucclProtoLL && chunk <= static_cast<size_t>(kLLBlocks) * kLLDataPerBlock && reducible(op.dtype))
        return chunkLL(c, op, chunk, KERN_RS_LL);
      return rsDirect(c, op, chunk, ch);
    case ucclCollBroadcast: return bcastDirect(c, op, chunk, ch);
    case ucclCollReduce: return reduceDirect(c, op, chunk, ch);
    case ucclCollAllToAll:
      if (ch.proto == ucclProtoLL && chunk <= static_cast<size_t>(kLLBlocks) * kLLDataPerBlock) return chunkLL(c, op, chunk, KERN_A2A_LL);
      return a2aDirect(c, op, chunk, ch);
    case ucclCollSendRecv: {
      std::vector<CollOp> v(1, op);
      return executeP2pBatch(c, v);
    }
    default: return ucclInternalError;
  }
}

}  // namespace uccl

// ------------------------------------------------------------------ point-to-point batches
namespace uccl {

ucclResult_t executeP2pBatch(Comm* c, const std::vector<CollOp>& ops) {
  if (ops.empty()) return ucclSuccess;
  size_t total = 0;
  for (const CollOp& op : ops) total += op.count * dataTypeSize(op.dtype);
  commCount(c, ucclCollSendRecv, total, c->backend == BACKEND_CPU || c->useNet ? ucclAlgoNet : ucclAlgoAuto);

  if (c->backend == BACKEND_CPU) {
    std::vector<HostP2pOp> v;
    for (const CollOp& op : ops) v.push_back({op.isSend, op.root, op.send, op.recv, op.count * dataTypeSize(op.dtype)});
    return hostSendRecv(c, v);
  }
  int prevDev = -1;
  cudaGetDevice(&prevDev);
  if (prevDev != c->cudaDev) cudaSetDevice(c->cudaDev);
  struct Restore {
    int d, cur;
    ~Restore() { if (d >= 0 && d != cur) cudaSetDevice(d); }
  } restore{prevDev, c->cudaDev};

  // self pairs are plain device copies
  std::vector<CollOp> rest;
  std::vector<bool> used(ops.size(), false);
  for (size_t i = 0; i < ops.size(); ++i) {
    if (used[i] || ops[i].root != c->rank) continue;
    if (!ops[i].isSend) continue;
    bool matched = false;
    for (size_t j = 0; j < ops.size(); ++j)
      if (!used[j] && j != i && ops[j].root == c->rank && !ops[j].isSend &&
          ops[j].count * dataTypeSize(ops[j].dtype) == ops[i].count * dataTypeSize(ops[i].dtype)) {
        ucclResult_t r = localCopy(c, ops[i].send, ops[j].recv, ops[i].count * dataTypeSize(ops[i].dtype), ops[i].stream);
        if (r != ucclSuccess) return r;
        used[i] = used[j] = true;
        matched = true;
        break;
      }
    if (!matched) {
      commSetError(c, "send to self without a matching recv in the same group");
      return ucclInvalidUsage;
    }
  }
  for (size_t i = 0; i < ops.size(); ++i) {
    if (used[i]) continue;
    if (ops[i].root == c->rank) {
      commSetError(c, "recv from self without a matching send in the same group");
      return ucclInvalidUsage;
    }
    rest.push_back(ops[i]);
  }
  if (rest.empty()) return ucclSuccess;

  if (c->useNet || !c->p2pReady) {
    return enqueueNetGpuP2p(c, rest);  // network path: staged through pinned host memory
  }

  // Operations with the same peer and direction share one FIFO: they form a chain that runs in
  // the order of the calls (two sends to one peer in a group are legal).  A launch carries the
  // next kP2pChainDepth operations of every chain, so both ends of a FIFO cut a long group at the
  // same places and no launch waits for an operation that its peer put into a later one.
  cudaStream_t stream = rest[0].stream;
  std::vector<std::vector<const CollOp*>> chains;
  std::vector<std::pair<int, bool>> keys;
  for (const CollOp& op : rest) {
    const std::pair<int, bool> key(c->peers[op.root].localRank, op.isSend);
    size_t k = 0;
    while (k < keys.size() && keys[k] != key) ++k;
    if (k == keys.size()) {
      keys.push_back(key);
      chains.emplace_back();
    }
    chains[k].push_back(&op);
  }
  if (chains.size() > static_cast<size_t>(kMaxP2pChains)) return ucclInternalError;
  size_t longest = 0;
  for (const auto& ch : chains) longest = std::max(longest, ch.size());
  for (size_t base = 0; base < longest; base += kP2pChainDepth) {
    P2pArgs a;
    memset(&a, 0, sizeof(a));
    a.dc = c->dev;
    int nops = 0;
    for (size_t k = 0; k < chains.size(); ++k) {
      int prev = -1;
      for (size_t i = base; i < std::min(chains[k].size(), base + kP2pChainDepth); ++i) {
        const CollOp& op = *chains[k][i];
        P2pOp& d = a.ops[nops];
        d.isSend = op.isSend ? 1 : 0;
        d.peer = keys[k].first;
        d.next = -1;
        d.src = static_cast<const char*>(op.send);
        d.dst = static_cast<char*>(op.recv);
        d.bytes = op.count * dataTypeSize(op.dtype);
        if (prev < 0) a.heads[a.nchains++] = nops;
        else a.ops[prev].next = nops;
        prev = nops++;
      }
    }
    cudaError_t e = launchP2pKernel(a, stream);
    if (e != cudaSuccess) {
      commSetError(c, "p2p kernel launch failed: %s", cudaGetErrorString(e));
      return ucclSystemError;
    }
  }
  return ucclSuccess;
}

}  // namespace uccl
