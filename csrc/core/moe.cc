// Host side of the MoE dispatch / combine pair: the context object that owns the symmetric
// receive area and the routing state, and the two launch entry points.
#include <string.h>

#include <algorithm>

#include "../kernels/moe.h"
#include "enqueue.h"
#include "log.h"

using namespace uccl;

struct ucclMoeContext {
  uint32_t magic = 0x4d4f4543;
  Comm* comm = nullptr;
  int maxTokens = 0, hidden = 0, experts = 0, topk = 0, rows = 0;
  SymSegment* seg = nullptr;   // receive area (multi-rank)
  char* localArea = nullptr;   // single-rank: plain device memory
  size_t offScale = 0, offMeta = 0, offCounts = 0, offArrived = 0, offOut = 0, total = 0;
  uint32_t* state = nullptr;   // device: sendCount[16] | ctasDone | epoch | overflow
  int32_t* slotOf = nullptr;   // device: [maxTokens][topk]
  int lastTokens = 0;
};

namespace {

bool ctxValid(const ucclMoeContext* m) { return m && m->magic == 0x4d4f4543 && commValid(m->comm); }

struct DeviceGuard {
  int prev = -1, want;
  explicit DeviceGuard(int dev) : want(dev) {
    cudaGetDevice(&prev);
    if (prev != want) cudaSetDevice(want);
  }
  ~DeviceGuard() {
    if (prev >= 0 && prev != want) cudaSetDevice(prev);
  }
};

size_t up256(size_t v) { return (v + 255) & ~size_t(255); }

void fillArgs(ucclMoeContext* m, MoeArgs* a) {
  Comm* c = m->comm;
  memset(a, 0, sizeof(*a));
  a->dc = c->dev;
  a->hidden = m->hidden;
  a->topk = m->topk;
  const int n = c->nRanks;
  a->expertsPerRank = m->experts / n;
  a->numExperts = m->experts;
  a->rowsPerSource = m->rows;
  if (n == 1) {
    a->dc.rank = 0;
    a->dc.nranks = 1;
  }
  for (int p = 0; p < n; ++p) {
    char* base = m->seg ? m->seg->peer[p] : m->localArea;
    a->recvX[p] = base;
    a->recvScale[p] = reinterpret_cast<float*>(base + m->offScale);
    a->recvMeta[p] = reinterpret_cast<int32_t*>(base + m->offMeta);
    a->recvCounts[p] = reinterpret_cast<int32_t*>(base + m->offCounts);
    a->arrived[p] = reinterpret_cast<uint32_t*>(base + m->offArrived);
    a->expertOut[p] = base + m->offOut;
  }
  a->sendCount = m->state;
  a->ctasDone = m->state + 16;
  a->epoch = m->state + 17;
  a->overflow = m->state + 18;
  a->slotOf = m->slotOf;
}

}  // namespace

extern "C" ucclResult_t ucclMoeCreate(ucclMoeContext_t* ctx, int maxTokensPerRank, int hidden, int numExperts, int topk,
                                      float capacityFactor, ucclComm_t comm) {
  Comm* c = toComm(comm);
  if (!commValid(c) || !ctx) return ucclInvalidArgument;
  *ctx = nullptr;
  if (c->backend != BACKEND_CUDA || (c->nRanks > 1 && (!c->p2pReady || c->useNet))) {
    commSetError(c, "MoE dispatch/combine needs all ranks in one NVLink domain");
    return ucclInvalidUsage;
  }
  const int n = c->nRanks;
  if (maxTokensPerRank <= 0 || hidden <= 0 || hidden % 128 != 0 || hidden > 8192 || topk < 1 || topk > 16 ||
      numExperts < n || numExperts % n != 0) {
    commSetError(c, "MoE shape not supported (hidden multiple of 128 up to 8192, topk <= 16, experts divisible by ranks)");
    return ucclInvalidArgument;
  }
  DeviceGuard guard(c->cudaDev);
  ucclMoeContext* m = new ucclMoeContext();
  m->comm = c;
  m->maxTokens = maxTokensPerRank;
  m->hidden = hidden;
  m->experts = numExperts;
  m->topk = topk;
  const long worst = static_cast<long>(maxTokensPerRank) * std::min(topk, numExperts / n);
  long rows = worst;
  if (capacityFactor > 0.f) {
    rows = static_cast<long>(capacityFactor * maxTokensPerRank * topk / n + 0.999f);
    rows = std::max(1L, std::min(rows, worst));
  }
  if (rows >= (1L << 24)) {
    delete m;
    return ucclInvalidArgument;
  }
  m->rows = static_cast<int>(rows);
  const size_t totalRows = static_cast<size_t>(n) * m->rows;
  m->offScale = up256(totalRows * hidden);
  m->offMeta = m->offScale + up256(totalRows * (hidden / 128) * sizeof(float));
  m->offCounts = m->offMeta + up256(totalRows * 4 * sizeof(int32_t));
  m->offArrived = m->offCounts + 256;
  m->offOut = m->offArrived + 256;
  m->total = m->offOut + up256(totalRows * hidden * 2);
  ucclResult_t r = ucclSuccess;
  if (n > 1) {
    r = c->heap.alloc(m->total, &m->seg);
    if (r == ucclSuccess && cudaMemset(m->seg->local + m->offCounts, 0, 512) != cudaSuccess) r = ucclSystemError;
  } else {
    void* p = nullptr;
    if (cudaMalloc(&p, m->total) != cudaSuccess) r = ucclSystemError;
    else cudaMemset(static_cast<char*>(p) + m->offCounts, 0, 512);
    m->localArea = static_cast<char*>(p);
  }
  void* st = nullptr;
  void* so = nullptr;
  if (r == ucclSuccess && (cudaMalloc(&st, 64 * sizeof(uint32_t)) != cudaSuccess ||
                           cudaMalloc(&so, static_cast<size_t>(maxTokensPerRank) * topk * sizeof(int32_t)) != cudaSuccess))
    r = ucclSystemError;
  if (r != ucclSuccess) {
    (void)cudaGetLastError();
    commSetError(c, "MoE context allocation failed (%zu bytes of symmetric memory)", m->total);
    if (m->seg) c->heap.release(m->seg);
    if (m->localArea) cudaFree(m->localArea);
    if (st) cudaFree(st);
    delete m;
    return r;
  }
  cudaMemset(st, 0, 64 * sizeof(uint32_t));
  cudaMemset(so, 0xff, static_cast<size_t>(maxTokensPerRank) * topk * sizeof(int32_t));
  cudaDeviceSynchronize();
  m->state = static_cast<uint32_t*>(st);
  m->slotOf = static_cast<int32_t*>(so);
  if (n > 1) c->bootstrap.barrier();
  *ctx = m;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclMoeDestroy(ucclMoeContext_t m) {
  if (!m) return ucclSuccess;
  if (!ctxValid(m)) return ucclInvalidArgument;
  Comm* c = m->comm;
  DeviceGuard guard(c->cudaDev);
  cudaDeviceSynchronize();
  if (c->nRanks > 1 && !c->abortFlag.load() && c->asyncError.load() == ucclSuccess) c->bootstrap.barrier();
  if (m->seg) c->heap.release(m->seg);
  if (m->localArea) cudaFree(m->localArea);
  cudaFree(m->state);
  cudaFree(m->slotOf);
  m->magic = 0;
  delete m;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclMoeGetLayout(ucclMoeContext_t m, ucclMoeLayout_t* l) {
  if (!ctxValid(m) || !l) return ucclInvalidArgument;
  char* base = m->seg ? m->seg->local : m->localArea;
  l->recvX = base;
  l->recvScale = reinterpret_cast<float*>(base + m->offScale);
  l->recvMeta = reinterpret_cast<int32_t*>(base + m->offMeta);
  l->recvCounts = reinterpret_cast<int32_t*>(base + m->offCounts);
  l->expertOut = base + m->offOut;
  l->rowsPerSource = m->rows;
  l->nranks = m->comm->nRanks;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclMoeDispatch(ucclMoeContext_t m, const void* x, const int32_t* topkIdx, int tokens,
                                        void* stream) {
  if (!ctxValid(m) || !x || !topkIdx || tokens < 0 || tokens > m->maxTokens) return ucclInvalidArgument;
  if (reinterpret_cast<uintptr_t>(x) & 15) return ucclInvalidArgument;
  Comm* c = m->comm;
  DeviceGuard guard(c->cudaDev);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // nobody writes into a receive area that its owner may still be reading from the last round
  if (c->nRanks > 1) {
    ucclResult_t r = enqueueBarrier(c, s);
    if (r != ucclSuccess) return r;
  }
  MoeArgs a;
  fillArgs(m, &a);
  a.tokens = tokens;
  a.x = x;
  a.topkIdx = topkIdx;
  m->lastTokens = tokens;
  commCount(c, ucclCollAllToAll, static_cast<size_t>(tokens) * m->topk * (m->hidden + m->hidden / 32), ucclAlgoTwoShot);
  if (launchMoeDispatch(a, s) != cudaSuccess) {
    commSetError(c, "MoE dispatch launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  return ucclSuccess;
}

extern "C" ucclResult_t ucclMoeCombine(ucclMoeContext_t m, const float* topkWeight, int tokens, void* out, void* stream) {
  if (!ctxValid(m) || !topkWeight || !out || tokens < 0 || tokens > m->maxTokens) return ucclInvalidArgument;
  if (reinterpret_cast<uintptr_t>(out) & 15) return ucclInvalidArgument;
  Comm* c = m->comm;
  DeviceGuard guard(c->cudaDev);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ucclResult_t r;
  // every rank's expert outputs are complete before anybody pulls them
  if (c->nRanks > 1 && (r = enqueueBarrier(c, s)) != ucclSuccess) return r;
  MoeArgs a;
  fillArgs(m, &a);
  a.tokens = tokens;
  a.topkWeight = topkWeight;
  a.out = out;
  commCount(c, ucclCollAllToAll, static_cast<size_t>(tokens) * m->topk * m->hidden * 2, ucclAlgoTwoShot);
  if (launchMoeCombine(a, s) != cudaSuccess) {
    commSetError(c, "MoE combine launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  // peers have finished pulling from this rank before expertOut is overwritten
  if (c->nRanks > 1 && (r = enqueueBarrier(c, s)) != ucclSuccess) return r;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclMoeOverflow(ucclMoeContext_t m, unsigned int* rows) {
  if (!ctxValid(m) || !rows) return ucclInvalidArgument;
  DeviceGuard guard(m->comm->cudaDev);
  if (cudaMemcpy(rows, m->state + 18, sizeof(uint32_t), cudaMemcpyDeviceToHost) != cudaSuccess) return ucclSystemError;
  return ucclSuccess;
}
