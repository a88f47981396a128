// Public collective entry points: argument validation, then direct execution or deferral into
// the current group.  The validation matrix follows the reference's front door
// (src/collectives.cc:29-125): invalid / aborted communicator, count == 0 succeeds without
// touching the buffers, null buffers, data type and reduction operator ranges.
#include <algorithm>
#include <vector>

#include "enqueue.h"
#include "log.h"

using namespace uccl;

namespace {

ucclResult_t validateComm(Comm* c) {
  if (!commValid(c)) return ucclInvalidArgument;
  if (c->abortFlag.load(std::memory_order_relaxed)) return ucclInvalidUsage;
  const int ae = c->asyncError.load(std::memory_order_relaxed);
  if (ae != ucclSuccess) return static_cast<ucclResult_t>(ae);
  return ucclSuccess;
}

bool dtypeOk(ucclDataType_t t) { return t >= 0 && t < ucclNumTypes; }
bool dtypeReducible(ucclDataType_t t) { return t == ucclFloat16 || t == ucclBfloat16 || t == ucclFloat32; }

ucclResult_t submit(CollOp& op, ucclComm_t comm, void* stream) {
  op.comm = toComm(comm);
  op.stream = static_cast<cudaStream_t>(stream);
  if (groupActive()) return groupAppend(op);
  return executeOp(op);
}

}  // namespace

extern "C" ucclResult_t ucclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ucclDataType_t datatype,
                                      ucclRedOp_t op, ucclComm_t comm, void* stream) {
  ucclResult_t r = validateComm(toComm(comm));
  if (r != ucclSuccess) return r;
  UCCL_LOG(TRACE, "ucclAllReduce count=%zu dtype=%d", count, (int)datatype);
  if (!dtypeOk(datatype) || op < 0 || op >= ucclNumOps) return ucclInvalidArgument;
  if (!dtypeReducible(datatype)) return ucclInvalidArgument;
  if (count == 0) return ucclSuccess;
  if (!sendbuff || !recvbuff) return ucclInvalidArgument;
  CollOp o;
  o.kind = ucclCollAllReduce;
  o.send = sendbuff;
  o.recv = recvbuff;
  o.count = count;
  o.dtype = datatype;
  return submit(o, comm, stream);
}

extern "C" ucclResult_t ucclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ucclDataType_t datatype,
                                      ucclComm_t comm, void* stream) {
  ucclResult_t r = validateComm(toComm(comm));
  if (r != ucclSuccess) return r;
  UCCL_LOG(TRACE, "ucclAllGather sendcount=%zu dtype=%d", sendcount, (int)datatype);
  if (!dtypeOk(datatype)) return ucclInvalidArgument;
  if (sendcount == 0) return ucclSuccess;
  if (!sendbuff || !recvbuff) return ucclInvalidArgument;
  CollOp o;
  o.kind = ucclCollAllGather;
  o.send = sendbuff;
  o.recv = recvbuff;
  o.count = sendcount;
  o.dtype = datatype;
  return submit(o, comm, stream);
}

extern "C" ucclResult_t ucclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount,
                                          ucclDataType_t datatype, ucclRedOp_t op, ucclComm_t comm, void* stream) {
  ucclResult_t r = validateComm(toComm(comm));
  if (r != ucclSuccess) return r;
  UCCL_LOG(TRACE, "ucclReduceScatter recvcount=%zu dtype=%d", recvcount, (int)datatype);
  if (!dtypeOk(datatype) || op < 0 || op >= ucclNumOps) return ucclInvalidArgument;
  if (!dtypeReducible(datatype)) return ucclInvalidArgument;
  if (recvcount == 0) return ucclSuccess;
  if (!sendbuff || !recvbuff) return ucclInvalidArgument;
  CollOp o;
  o.kind = ucclCollReduceScatter;
  o.send = sendbuff;
  o.recv = recvbuff;
  o.count = recvcount;
  o.dtype = datatype;
  return submit(o, comm, stream);
}

extern "C" ucclResult_t ucclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ucclDataType_t datatype,
                                      int root, ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  ucclResult_t r = validateComm(c);
  if (r != ucclSuccess) return r;
  if (!dtypeOk(datatype) || root < 0 || root >= c->nRanks) return ucclInvalidArgument;
  if (count == 0) return ucclSuccess;
  if (!recvbuff || (c->rank == root && !sendbuff)) return ucclInvalidArgument;
  CollOp o;
  o.kind = ucclCollBroadcast;
  o.send = sendbuff ? sendbuff : recvbuff;
  o.recv = recvbuff;
  o.count = count;
  o.dtype = datatype;
  o.root = root;
  return submit(o, comm, stream);
}

extern "C" ucclResult_t ucclReduce(const void* sendbuff, void* recvbuff, size_t count, ucclDataType_t datatype,
                                   ucclRedOp_t op, int root, ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  ucclResult_t r = validateComm(c);
  if (r != ucclSuccess) return r;
  if (!dtypeOk(datatype) || op < 0 || op >= ucclNumOps || root < 0 || root >= c->nRanks) return ucclInvalidArgument;
  if (!dtypeReducible(datatype)) return ucclInvalidArgument;
  if (count == 0) return ucclSuccess;
  if (!sendbuff || (c->rank == root && !recvbuff)) return ucclInvalidArgument;
  CollOp o;
  o.kind = ucclCollReduce;
  o.send = sendbuff;
  o.recv = recvbuff;
  o.count = count;
  o.dtype = datatype;
  o.root = root;
  return submit(o, comm, stream);
}

extern "C" ucclResult_t ucclAllToAll(const void* sendbuff, void* recvbuff, size_t count, ucclDataType_t datatype,
                                     ucclComm_t comm, void* stream) {
  ucclResult_t r = validateComm(toComm(comm));
  if (r != ucclSuccess) return r;
  if (!dtypeOk(datatype)) return ucclInvalidArgument;
  if (count == 0) return ucclSuccess;
  if (!sendbuff || !recvbuff || sendbuff == recvbuff) return ucclInvalidArgument;
  CollOp o;
  o.kind = ucclCollAllToAll;
  o.send = sendbuff;
  o.recv = recvbuff;
  o.count = count;
  o.dtype = datatype;
  return submit(o, comm, stream);
}

extern "C" ucclResult_t ucclSend(const void* sendbuff, size_t count, ucclDataType_t datatype, int peer,
                                 ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  ucclResult_t r = validateComm(c);
  if (r != ucclSuccess) return r;
  if (!dtypeOk(datatype) || peer < 0 || peer >= c->nRanks) return ucclInvalidArgument;
  if (count == 0) return ucclSuccess;
  if (!sendbuff) return ucclInvalidArgument;
  CollOp o;
  o.kind = ucclCollSendRecv;
  o.isSend = true;
  o.send = sendbuff;
  o.count = count;
  o.dtype = datatype;
  o.root = peer;
  return submit(o, comm, stream);
}

extern "C" ucclResult_t ucclRecv(void* recvbuff, size_t count, ucclDataType_t datatype, int peer, ucclComm_t comm,
                                 void* stream) {
  Comm* c = toComm(comm);
  ucclResult_t r = validateComm(c);
  if (r != ucclSuccess) return r;
  if (!dtypeOk(datatype) || peer < 0 || peer >= c->nRanks) return ucclInvalidArgument;
  if (count == 0) return ucclSuccess;
  if (!recvbuff) return ucclInvalidArgument;
  CollOp o;
  o.kind = ucclCollSendRecv;
  o.isSend = false;
  o.recv = recvbuff;
  o.count = count;
  o.dtype = datatype;
  o.root = peer;
  return submit(o, comm, stream);
}

extern "C" ucclResult_t ucclCommQueryTuning(ucclComm_t comm, ucclCollKind_t coll, size_t bytes, int symmetric,
                                            ucclAlgo_t* algo, ucclProto_t* proto, int* nChannels) {
  Comm* c = toComm(comm);
  if (!commValid(c) || coll < 0 || coll > ucclCollRma) return ucclInvalidArgument;
  const bool nvls = c->arena && c->arena->mc;
  TuneChoice ch = chooseFor(c, coll, bytes, symmetric != 0, nvls, ucclBfloat16);
  if (algo) *algo = ch.algo;
  if (proto) *proto = ch.proto;
  if (nChannels) *nChannels = ch.blocks;
  return ucclSuccess;
}

// Canaries (UCCL_CANARY=1).  A buffer from ucclMemAlloc then sits between two painted regions of
// its own mapping: kCanaryBytes in front, and everything from its end to the end of the mapping
// (at least kCanaryBytes, checked up to kCanaryTailMax) behind.  A store that misses the buffer by
// a little -- this rank's or a peer's, through the peer or the multicast alias -- lands there
// instead of in a neighbour, and ucclMemCheck / ucclMemFree find it.  Stores that miss by more than
// the mapping reach unmapped addresses, which the hardware reports.
static constexpr size_t kCanaryBytes = 4096;
static constexpr size_t kCanaryTailMax = 64u << 10;
static constexpr unsigned char kCanaryByte = 0xC5;

static size_t canaryTail(const SymSegment* seg) {
  return std::min(kCanaryTailMax, seg->mapSize - seg->guard - seg->userSize);
}

static void paintCanaries(SymSegment* seg) {
  cudaMemset(seg->local, kCanaryByte, seg->guard);
  cudaMemset(seg->local + seg->guard + seg->userSize, kCanaryByte, canaryTail(seg));
  cudaDeviceSynchronize();
}

// Offset (relative to the caller's pointer; negative = in front) of the first overwritten canary
// byte of `seg`, or false when both canaries are intact.
static bool canaryBroken(const SymSegment* seg, long long* where) {
  if (!seg->guard) return false;
  const size_t tail = canaryTail(seg);
  std::vector<unsigned char> h(seg->guard + tail);
  if (cudaMemcpy(h.data(), seg->local, seg->guard, cudaMemcpyDeviceToHost) != cudaSuccess ||
      cudaMemcpy(h.data() + seg->guard, seg->local + seg->guard + seg->userSize, tail, cudaMemcpyDeviceToHost) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  for (size_t i = 0; i < h.size(); ++i)
    if (h[i] != kCanaryByte) {
      *where = i < seg->guard ? static_cast<long long>(i) - static_cast<long long>(seg->guard)
                              : static_cast<long long>(seg->userSize + (i - seg->guard));
      return true;
    }
  return false;
}

extern "C" ucclResult_t ucclMemCheck(ucclComm_t comm) {
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  if (!c->p2pReady || !c->cfg.canary) return ucclSuccess;
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != c->cudaDev) cudaSetDevice(c->cudaDev);
  cudaDeviceSynchronize();
  c->bootstrap.barrier();  // every rank's stores into my buffers have landed
  ucclResult_t r = ucclSuccess;
  for (SymSegment* seg : c->heap.segments()) {
    long long where = 0;
    if (canaryBroken(seg, &where)) {
      commSetError(c, "memory check: buffer %p (%zu bytes) has a store outside its bounds at byte offset %lld",
                   static_cast<void*>(seg->local + seg->guard), seg->userSize, where);
      r = ucclInternalError;
      break;
    }
  }
  if (prev != c->cudaDev && prev >= 0) cudaSetDevice(prev);
  return r;
}

extern "C" ucclResult_t ucclMemAlloc(void** ptr, size_t size, ucclComm_t comm) {
  Comm* c = toComm(comm);
  if (!commValid(c) || !ptr || size == 0) return ucclInvalidArgument;
  *ptr = nullptr;
  if (c->backend != BACKEND_CUDA) {
    commSetError(c, "ucclMemAlloc needs a communicator on GPUs");
    return ucclInvalidUsage;
  }
  if (!c->p2pReady) {
    // no NVLink domain: hand out ordinary device memory so that callers keep working
    void* p = nullptr;
    if (cudaMalloc(&p, size) != cudaSuccess) return ucclSystemError;
    *ptr = p;
    return ucclSuccess;
  }
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != c->cudaDev) cudaSetDevice(c->cudaDev);
  SymSegment* seg = nullptr;
  const size_t guard = c->cfg.canary ? kCanaryBytes : 0;
  ucclResult_t r = c->heap.alloc(size + 2 * guard, &seg);
  if (r == ucclSuccess) {
    seg->guard = guard;
    seg->userSize = size;
    if (guard) paintCanaries(seg);
  }
  if (prev != c->cudaDev && prev >= 0) cudaSetDevice(prev);
  if (r != ucclSuccess) return r;
  *ptr = seg->local + guard;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclMemFree(void* ptr, ucclComm_t comm) {
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  if (!ptr) return ucclSuccess;
  if (!c->p2pReady) {
    cudaFree(ptr);
    return ucclSuccess;
  }
  SymSegment* seg = c->heap.find(ptr, 1);
  if (!seg || seg->local + seg->guard != ptr || seg == c->arena) return ucclInvalidArgument;
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != c->cudaDev) cudaSetDevice(c->cudaDev);
  cudaDeviceSynchronize();
  c->bootstrap.barrier();  // peers may still be reading this memory
  long long where = 0;
  const bool broken = canaryBroken(seg, &where);
  if (broken)
    commSetError(c, "memory check: buffer %p (%zu bytes) was freed with a store outside its bounds at byte offset %lld",
                 ptr, seg->userSize, where);
  ucclResult_t r = c->heap.release(seg);
  if (prev != c->cudaDev && prev >= 0) cudaSetDevice(prev);
  return broken && r == ucclSuccess ? ucclInternalError : r;
}

extern "C" ucclResult_t ucclMemPeerPointer(const void* ptr, int peer, ucclComm_t comm, void** peerPtr) {
  Comm* c = toComm(comm);
  if (!commValid(c) || !peerPtr || peer < 0 || peer >= c->nRanks) return ucclInvalidArgument;
  *peerPtr = nullptr;
  if (!c->p2pReady) return ucclSuccess;
  SymSegment* seg = c->heap.find(ptr, 1);
  if (!seg) return ucclSuccess;
  const int lp = c->peers[peer].localRank;
  *peerPtr = seg->peer[lp] + (static_cast<const char*>(ptr) - seg->local);
  return ucclSuccess;
}

extern "C" ucclResult_t ucclMemMulticastPointer(const void* ptr, ucclComm_t comm, void** mcPtr) {
  Comm* c = toComm(comm);
  if (!commValid(c) || !mcPtr) return ucclInvalidArgument;
  *mcPtr = nullptr;
  if (!c->p2pReady) return ucclSuccess;
  SymSegment* seg = c->heap.find(ptr, 1);
  if (!seg || !seg->mc) return ucclSuccess;
  *mcPtr = seg->mc + (static_cast<const char*>(ptr) - seg->local);
  return ucclSuccess;
}
