// Fused compute + collective entry points: all-reduce + residual + RMSNorm, all-gather -> GEMM,
// GEMM -> reduce-scatter.  None of them exists in the reference; they are the tensor-parallel
// building blocks the library is benchmarked on (a Llama-style MLP block: sequence-parallel
// activations are gathered in front of the column-parallel up/gate projection and the
// row-parallel down projection ends in a reduce-scatter).
#include <stdlib.h>
#include <string.h>
#include <strings.h>

#include <algorithm>

#include "../kernels/collectives.cuh"
#include "../kernels/gemm_sm100.h"
#include "enqueue.h"
#include "log.h"

using namespace uccl;

namespace {

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

ucclResult_t validate(Comm* c) {
  if (!commValid(c)) return ucclInvalidArgument;
  if (c->abortFlag.load()) return ucclInvalidUsage;
  const int ae = c->asyncError.load();
  if (ae != ucclSuccess) return static_cast<ucclResult_t>(ae);
  if (c->backend != BACKEND_CUDA) {
    commSetError(c, "fused kernels need a communicator on GPUs");
    return ucclInvalidUsage;
  }
  if (c->nRanks > 1 && (!c->p2pReady || c->useNet)) {
    commSetError(c, "fused kernels need all ranks in one NVLink domain");
    return ucclInvalidUsage;
  }
  return ucclSuccess;
}

// CTAs that run the communication role of a fused GEMM launch: UCCL_FUSED_COMM_CTAS, else the
// communicator's option, else 8.
int fusedCommCtas(Comm* c) {
  const char* s = getenv("UCCL_FUSED_COMM_CTAS");
  if (s && *s) {
    const int v = atoi(s);
    if (v >= 1 && v <= 64) return v;
  }
  if (c->fusedCommCtas > 0) return c->fusedCommCtas;
  return c->cfg.maxCtas > 0 ? std::min(c->cfg.maxCtas, 32) : 8;
}

// How the all-gather of the all-gather -> GEMM fusion moves its rows:
//   1 copy engines next to the GEMM (default: no SM work at all),
//   2 dedicated communication CTAs inside the launch,
//   3 "spread": a forwarder warp in every GEMM CTA.
// UCCL_FUSED_AG=ce|kernel|spread wins over ucclCommSetFusedOptions; an SM algorithm forced on the
// communicator selects 3.
int fusedAgMode(Comm* c) {
  const char* s = getenv("UCCL_FUSED_AG");
  if (s && *s) {
    if (!strcasecmp(s, "ce") || !strcasecmp(s, "copy_engine")) return 1;
    if (!strcasecmp(s, "kernel") || !strcasecmp(s, "ctas")) return 2;
    if (!strcasecmp(s, "spread")) return 3;
  }
  if (c->fusedAgMode != 0) return c->fusedAgMode;
  if (c->forcedAlgo == ucclAlgoOneShot || c->forcedAlgo == ucclAlgoTwoShot || c->forcedAlgo == ucclAlgoRing) return 3;
  return 1;
}

// UCCL_FUSED_SELF=1 runs the fused kernels on a one-rank communicator too (every "peer" is this
// GPU): the whole data path of the fusion in a single process, for profiling one kernel alone.
bool fusedSelf() {
  const char* s = getenv("UCCL_FUSED_SELF");
  return s && atoi(s) != 0;
}

// UCCL_FUSED_FOLD_BARRIER=0 runs the rank barrier of a fused launch as a kernel of its own in
// front of it (the older arrangement) instead of inside the GEMM kernel's prologue.
bool foldBarrier() {
  const char* s = getenv("UCCL_FUSED_FOLD_BARRIER");
  return !(s && *s && atoi(s) == 0);
}

struct Sym {
  SymSegment* seg = nullptr;
  size_t off = 0;
};
bool symOf(Comm* c, const void* p, size_t bytes, Sym* out) {
  if (!c->p2pReady || (reinterpret_cast<uintptr_t>(p) & 15)) return false;
  SymSegment* s = c->heap.find(p, bytes);
  if (!s) return false;
  out->seg = s;
  out->off = static_cast<size_t>(static_cast<const char*>(p) - s->local);
  return true;
}

}  // namespace

extern "C" ucclResult_t ucclAllReduceResidualRMSNorm(const void* x, const void* residual, const void* gamma, void* out,
                                                     void* residualOut, int tokens, int hidden, float eps,
                                                     ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  ucclResult_t r = validate(c);
  if (r != ucclSuccess) return r;
  if (!x || !residual || !gamma || !out || !residualOut || tokens <= 0 || hidden <= 0) return ucclInvalidArgument;
  if (hidden % 8 != 0 || hidden > 16384) {
    commSetError(c, "hidden must be a multiple of 8 and at most 16384");
    return ucclInvalidArgument;
  }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(gamma) |
       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residualOut)) & 15)
    return ucclInvalidArgument;
  DeviceGuard guard(c->cudaDev);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t bytes = static_cast<size_t>(tokens) * hidden * 2;
  const int n = c->localRanks;
  ArNormArgs a;
  memset(&a, 0, sizeof(a));
  a.dc = c->dev;
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.gamma = static_cast<const __nv_bfloat16*>(gamma);
  a.outLocal = static_cast<char*>(out);
  a.tokens = tokens;
  a.hidden = hidden;
  a.eps = eps;
#ifdef UCCL_EXPERIMENTS
  {
    const char* dbg = getenv("UCCL_NORM_DEBUG");
    a.debug = dbg ? atoi(dbg) : 0;
  }
#endif
  // rows per pass of the all-reduce phase on the switch path; 0 = normalise own rows from registers
  // (8 ranks, 8192 x 8192: 403-499 us with one row per pass, 511-519 in one phase, 526-552 with two or four rows)
  a.mcRows = c->fusedNormRows >= 0 ? c->fusedNormRows : 1;
  if (const char* e = getenv("UCCL_NORM_MC_ROWS")) a.mcRows = atoi(e);
  if (a.mcRows < 0 || a.mcRows > 4) a.mcRows = 1;
  commCount(c, ucclCollAllReduce, bytes, c->arena && c->arena->mc ? ucclAlgoNvls : ucclAlgoTwoShot);
  if (c->nRanks == 1) {
    a.dc.nranks = 1;
    a.inUser = static_cast<const char*>(x);
    a.resOutUser = static_cast<char*>(residualOut);
    const int blocks = std::min(deviceSmCount(), std::max(1, tokens));
    if (launchArNormKernel(a, blocks, s) != cudaSuccess) {
      commSetError(c, "norm kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
      return ucclSystemError;
    }
    return ucclSuccess;
  }
  const size_t stageOff = stagingOffset(c);
  const size_t half = ((c->cfg.stagingBytes & ~size_t(4095)) / 2) & ~size_t(255);
  Sym sx, sr;
  const bool symX = symOf(c, x, bytes, &sx);
  const bool symR = symOf(c, residualOut, bytes, &sr);
  if ((!symX || !symR) && bytes > half) {
    commSetError(c, "tensor of %zu bytes does not fit the staging area; allocate x and residual_out with ucclMemAlloc "
                    "or raise UCCL_STAGING_BYTES", bytes);
    return ucclInvalidUsage;
  }
  for (int p = 0; p < n; ++p) {
    a.in[p] = symX ? sx.seg->peer[p] + sx.off : c->arena->peer[p] + stageOff;
    a.resOut[p] = symR ? sr.seg->peer[p] + sr.off : c->arena->peer[p] + stageOff + half;
  }
  if (symX) a.inMc = sx.seg->mc ? sx.seg->mc + sx.off : nullptr;
  else {
    a.inMc = c->arena->mc ? c->arena->mc + stageOff : nullptr;
    a.inUser = static_cast<const char*>(x);
  }
  if (symR) a.resOutMc = sr.seg->mc ? sr.seg->mc + sr.off : nullptr;
  else {
    a.resOutMc = c->arena->mc ? c->arena->mc + stageOff + half : nullptr;
    a.resOutUser = static_cast<char*>(residualOut);
  }
  if (c->forcedAlgo == ucclAlgoTwoShot || c->forcedAlgo == ucclAlgoOneShot) a.inMc = nullptr, a.resOutMc = nullptr;
  // between two GPUs the switch has nothing to reduce or replicate, and plain peer loads / stores
  // measured 1.7x faster than multimem there (369 us against 630 us for 8192 x 8192)
  if (n <= 2 && c->forcedAlgo != ucclAlgoNvls) a.inMc = nullptr, a.resOutMc = nullptr;
  int blocks = c->cfg.maxCtas > 0 ? std::min(c->cfg.maxCtas, kMaxBlocks) : kMaxBlocks;
  if (c->forcedBlocks > 0) blocks = std::min(c->forcedBlocks, kMaxBlocks);
  blocks = std::min(blocks, std::max(1, (tokens + n - 1) / n));
  if (launchArNormKernel(a, blocks, s) != cudaSuccess) {
    commSetError(c, "fused norm kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  return ucclSuccess;
}

extern "C" ucclResult_t ucclAllGatherGemm(const void* xShard, void* xFull, const void* W, void* C, int M, int N, int K,
                                          int epilogue, ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  ucclResult_t r = validate(c);
  if (r != ucclSuccess) return r;
  if (!xShard || !xFull || !W || !C || M <= 0 || N <= 0 || K <= 0 || (epilogue != 0 && epilogue != 1))
    return ucclInvalidArgument;
  DeviceGuard guard(c->cudaDev);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int n = c->localRanks;
  GemmLaunch g;
  g.A = xFull;
  g.B = W;
  g.C = C;
  g.M = M;
  g.N = N;
  g.K = K;
  g.lda = K;
  g.ldb = K;
  g.ldc = epilogue == 1 ? N / 2 : N;
  g.epilogue = epilogue;
  g.err = c->hostFlagsDev + 16;
  if (c->nRanks == 1 && !fusedSelf()) {
    g.A = xShard;
    return launchGemmBf16(g, nullptr, s);
  }
  if (M % n != 0 || (M / n) % 128 != 0) {
    commSetError(c, "all-gather GEMM needs M / nranks to be a multiple of 128 (M=%d, nranks=%d)", M, n);
    return ucclInvalidArgument;
  }
  if (M / 128 + 2 > kGemmMaxRowBlocks) return ucclInvalidArgument;  // two more lines hold the launch's go flag and work counter
  Sym sf;
  if (!symOf(c, xFull, static_cast<size_t>(M) * K * 2, &sf)) {
    commSetError(c, "xFull must come from ucclMemAlloc");
    return ucclInvalidArgument;
  }
  const int rows = M / n;
  const size_t shardBytes = static_cast<size_t>(rows) * K * 2;
  const char* myRows = static_cast<const char*>(xFull) + static_cast<size_t>(c->localRank) * shardBytes;
  if (reinterpret_cast<uintptr_t>(xShard) & 15) return ucclInvalidArgument;
  // Arrival counters start at zero.  The barrier orders the zeroing before any rank's pushes, and
  // those pushes after every rank's previous readers of its xFull.
  // With copy engines the pushes start from the host side, so the barrier stays a kernel of its own;
  // otherwise it runs inside the GEMM launch (the word after the last counter is its `go` flag).
  uint32_t* ready = reinterpret_cast<uint32_t*>(c->arena->local + kArenaGemmReadyOff);
  if (cudaMemsetAsync(ready, 0, kGemmFlagStrideBytes * (M / 128 + 1), s) != cudaSuccess) return ucclSystemError;
  const bool fold = foldBarrier() && fusedAgMode(c) != 1;
  if (!fold && (r = enqueueBarrier(c, s)) != ucclSuccess) return r;
  GemmFusion f;
  if (fold) {
    f.arena_peer = c->dev.arena;
    f.epochs = c->dev.epochs;
    f.go = ready + static_cast<size_t>(M / 128) * (kGemmFlagStrideBytes / 4);
  }
  f.role = 1;
  f.rank = c->localRank;
  f.nranks = n;
  f.comm_ctas = fusedCommCtas(c);
  f.timeout_ns = c->dev.timeoutNs;
  f.abort_flag = c->dev.abortFlag;
  f.rows_per_rank = rows;
  f.a_shard = xShard;
  f.a_inplace = myRows == static_cast<const char*>(xShard) ? 1 : 0;
  for (int p = 0; p < n; ++p) {
    f.a_full_peer[p] = sf.seg->peer[p] + sf.off;
    f.ready_peer[p] = reinterpret_cast<uint32_t*>(c->arena->peer[p] + kArenaGemmReadyOff);
  }
  // Two ways to move the rows: communication CTAs inside the GEMM launch (default), or copy
  // engines on side streams next to it (UCCL_FUSED_AG=ce, or algorithm copy_engine forced).
  const int agMode = fusedAgMode(c);
  if (agMode == 1) {
    commCount(c, ucclCollAllGather, static_cast<size_t>(M) * K * 2, ucclAlgoCopyEngine);
    f.a_external = 1;
    char* fullPeer[UCCL_MAX_LOCAL_RANKS];
    char* readyPeer[UCCL_MAX_LOCAL_RANKS];
    for (int p = 0; p < n; ++p) {
      fullPeer[p] = static_cast<char*>(f.a_full_peer[p]);
      readyPeer[p] = reinterpret_cast<char*>(f.ready_peer[p]);
    }
    // copy-engine lanes: UCCL_FUSED_CE_LANES, else the communicator's option (its commCtas field);
    // without either, one lane when there are several peers (measured at TP8: 415 us with one lane,
    // 530 us with two, 559 us with a stream per peer)
    int lanes = c->fusedAgMode == 0 ? (n > 2 ? 1 : 0) : c->fusedCommCtas;
    if (const char* e = getenv("UCCL_FUSED_CE_LANES")) lanes = atoi(e);
    if (lanes < 0 || n <= 2) lanes = 0;
    f.a_peer_major = lanes > 0 ? 1 : 0;
    if ((r = allGatherPushBegin(c, xShard, fullPeer, readyPeer, shardBytes, rows / 128, !f.a_inplace, lanes, s)) != ucclSuccess)
      return r;
    if ((r = launchGemmBf16(g, &f, s)) != ucclSuccess) return r;
    return allGatherPushEnd(c, !f.a_inplace, lanes, s);
  }
  commCount(c, ucclCollAllGather, static_cast<size_t>(M) * K * 2, ucclAlgoOneShot);
  f.a_spread = agMode == 3 ? 1 : 0;
  // The kernel reads my rows from the shard; a copy engine puts them into xFull meanwhile.
  const bool sideCopy = !f.a_inplace;
  if (sideCopy && (r = sideCopyBegin(c, const_cast<char*>(myRows), xShard, shardBytes, s)) != ucclSuccess) return r;
  if ((r = launchGemmBf16(g, &f, s)) != ucclSuccess) return r;
  if (sideCopy) return sideCopyEnd(c, s);
  return ucclSuccess;
}

extern "C" ucclResult_t ucclGemmReduceScatter(const void* A, const void* W, void* cPartial, void* out, int M, int N,
                                              int K, ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  ucclResult_t r = validate(c);
  if (r != ucclSuccess) return r;
  if (!A || !W || !cPartial || !out || M <= 0 || N <= 0 || K <= 0) return ucclInvalidArgument;
  DeviceGuard guard(c->cudaDev);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int n = c->localRanks;
  GemmLaunch g;
  g.A = A;
  g.B = W;
  g.C = cPartial;
  g.M = M;
  g.N = N;
  g.K = K;
  g.lda = K;
  g.ldb = K;
  g.ldc = N;
  g.err = c->hostFlagsDev + 16;
  if (c->nRanks == 1 && !fusedSelf()) {
    g.C = out;
    return launchGemmBf16(g, nullptr, s);
  }
  if (M % n != 0 || (M / n) % 128 != 0 || N % 8 != 0) {
    commSetError(c, "GEMM reduce-scatter needs M / nranks to be a multiple of 128 and N a multiple of 8");
    return ucclInvalidArgument;
  }
  if (M / 128 + 2 > kGemmMaxRowBlocks) return ucclInvalidArgument;  // two more lines hold the launch's go flag and work counter
  Sym sp;
  if (!symOf(c, cPartial, static_cast<size_t>(M) * N * 2, &sp)) {
    commSetError(c, "cPartial must come from ucclMemAlloc");
    return ucclInvalidArgument;
  }
  // cPartial is the staging buffer of this rank: slot s ([rows_per_rank, N]) receives rank s's
  // partial sums of this rank's rows.  The counters start at zero, and the barrier also orders
  // this launch's remote writes after every rank's previous use of its staging buffer.
  uint32_t* done = reinterpret_cast<uint32_t*>(c->arena->local + kArenaGemmDoneOff);
  if (cudaMemsetAsync(done, 0, kGemmFlagStrideBytes * (M / 128 + 2), s) != cudaSuccess) return ucclSystemError;
  const bool fold = foldBarrier();
  // the two lines after the last counter: the launch's go flag and the work counter of its summing tail
  uint32_t* go = done + static_cast<size_t>(M / 128) * (kGemmFlagStrideBytes / 4);
  uint32_t* tailNext = go + kGemmFlagStrideBytes / 4;
  // CTAs that only sum (UCCL_FUSED_RS_REDUCERS, else the communicator's option): when the links, not
  // the tensor cores, set the pace of the main loop, a few SMs taken from the GEMM cost nothing and
  // the summing no longer waits for the last tile
  int reducers = c->fusedRsReducers;
  if (const char* e = getenv("UCCL_FUSED_RS_REDUCERS")) reducers = atoi(e);
  if (reducers < 0 || reducers > 64) reducers = 0;
  if (!fold && (r = enqueueBarrier(c, s)) != ucclSuccess) return r;
  GemmFusion f;
  if (fold) {
    f.arena_peer = c->dev.arena;
    f.epochs = c->dev.epochs;
    f.go = go;
  }
  f.role = 2;
  f.tail_next = tailNext;
  f.rs_reducers = reducers;
  f.rank = c->localRank;
  f.nranks = n;
  f.timeout_ns = c->dev.timeoutNs;
  f.abort_flag = c->dev.abortFlag;
  f.rows_per_rank = M / n;
  for (int p = 0; p < n; ++p) {
    f.stage_peer[p] = sp.seg->peer[p] + sp.off;
    f.done_peer[p] = reinterpret_cast<uint32_t*>(c->arena->peer[p] + kArenaGemmDoneOff);
  }
  f.rs_out = out;
  f.rs_ldo = N;
  commCount(c, ucclCollReduceScatter, static_cast<size_t>(M) * N * 2, ucclAlgoOneShot);
  // When the kernel ends, every partial tile for this rank has arrived and been summed, and this
  // rank's own stores to its peers are complete: nothing is in flight in either direction.
  return launchGemmBf16(g, &f, s);
}
