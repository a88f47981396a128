// Launchers for the tcgen05 GEMM: tensor-map construction, grid sizing, template dispatch.
#include "gemm_sm100.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>

#include <algorithm>

#include "../core/cuda_driver.h"
#include "../core/log.h"
#include "device_comm.h"
#include "gemm_sm100.cuh"

namespace uccl {

int deviceSmCount() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

namespace {

// bf16 matrix [rows, cols] (row stride ld elements), 128-byte swizzled boxes of box_cols x box_rows.
bool makeTensorMap(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
                   uint32_t box_rows) {
  const DriverApi& d = driverApi();
  if (!d.ok) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = d.tensorMapEncodeTiled(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                                      box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    UCCL_LOG(ERROR, "cuTensorMapEncodeTiled failed: %s (base=%p rows=%llu cols=%llu ld=%llu)", driverErrorString(r),
             base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld);
    return false;
  }
  return true;
}

// Raises the dynamic shared-memory limit of one kernel once per (thread, device). The caller owns
// the two state words, one pair per kernel: kernels of equal signature share a function type.
template <typename Kern>
cudaError_t ensureSmem(Kern kern, int* last_dev, cudaError_t* err) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != *last_dev) {
    *err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::SMEM_BYTES);
    *last_dev = dev;
  }
  return *err;
}

template <int EPI, int COMM>
cudaError_t launchT(const CUtensorMap& tmA, const CUtensorMap& tmB, const gemm::PeerMaps& pm, const gemm::Args& args,
                    int grid, cudaStream_t stream) {
  const int threads = (COMM == gemm::kCommAllGather && args.a_spread) ? gemm::NUM_THREADS_FWD : gemm::NUM_THREADS;
  auto kern = gemm::gemm_bf16_kernel<EPI, COMM>;
  static thread_local int last_dev = -1;
  static thread_local cudaError_t attr_err = cudaSuccess;
  cudaError_t e = ensureSmem(kern, &last_dev, &attr_err);
  if (e != cudaSuccess) return e;
  kern<<<grid, threads, gemm::SMEM_BYTES, stream>>>(tmA, tmB, pm, args);
  return cudaGetLastError();
}

template <int EPI, int COMM>
cudaError_t launchPairT(const CUtensorMap& tmA, const CUtensorMap& tmB, const gemm::PeerMaps& pm,
                        const gemm::Args& args, int grid, cudaStream_t stream) {
  const int threads = (COMM == gemm::kCommAllGather && args.a_spread) ? gemm::NUM_THREADS_FWD : gemm::NUM_THREADS;
  auto kern = gemm::gemm2_bf16_kernel<EPI, COMM>;
  static thread_local int last_dev = -1;
  static thread_local cudaError_t attr_err = cudaSuccess;
  cudaError_t e = ensureSmem(kern, &last_dev, &attr_err);
  if (e != cudaSuccess) return e;
  kern<<<grid, threads, gemm::SMEM_BYTES, stream>>>(tmA, tmB, pm, args);
  return cudaGetLastError();
}

// Clusters of two CTAs that fit on the device at once (one CTA per SM; GPCs with an odd number of
// usable SMs leave one SM unpaired).
int maxResidentPairs() {
  static int cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return deviceSmCount() / 2;
  if (cached[dev] == 0) {
    auto kern = gemm::gemm2_bf16_kernel<gemm::kEpiStore, gemm::kCommNone>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::SMEM_BYTES);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * deviceSmCount(), 1, 1);
    cfg.blockDim = dim3(gemm::NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = gemm::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = deviceSmCount() / 2 - 4;
    }
    cached[dev] = n;
    UCCL_LOG(INFO, "gemm: %d CTA pairs can be resident on device %d", n, dev);
  }
  return cached[dev];
}

// UCCL_GEMM_PAIR=0 selects the single-CTA kernel, 1 the CTA-pair kernel (default).
bool usePairKernel() {
  const char* s = getenv("UCCL_GEMM_PAIR");
  return (s && *s) ? atoi(s) != 0 : true;
}

}  // namespace

ucclResult_t launchGemmBf16(const GemmLaunch& g, const GemmFusion* f, cudaStream_t stream) {
  if (!g.A || !g.B || !g.C || g.M <= 0 || g.N <= 0 || g.K <= 0) return ucclInvalidArgument;
  if (g.K % 8 != 0 || g.lda % 8 != 0 || g.ldb % 8 != 0 || g.ldc % 8 != 0) return ucclInvalidArgument;
  if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B) | reinterpret_cast<uintptr_t>(g.C)) & 15)
    return ucclInvalidArgument;
  if (g.epilogue == gemm::kEpiSwiGLU && (g.N % 2 != 0)) return ucclInvalidArgument;
  const int role = f ? f->role : 0;
  if (role == gemm::kCommReduceScatter && g.epilogue != gemm::kEpiStore)
    return ucclInvalidArgument;

  CUtensorMap tmA, tmB;
  if (!makeTensorMap(&tmA, g.A, g.M, g.K, g.lda, gemm::BK, gemm::BM)) return ucclSystemError;
  if (!makeTensorMap(&tmB, g.B, g.N, g.K, g.ldb, gemm::BK, gemm::BN / 2)) return ucclSystemError;

  gemm::Args a = {};
  a.M = g.M;
  a.N = g.N;
  a.K = g.K;
  a.C = static_cast<__nv_bfloat16*>(g.C);
  a.ldc = g.ldc;
  a.tiles_m = (g.M + gemm::BM - 1) / gemm::BM;
  if (g.epilogue == gemm::kEpiSwiGLU) {
    a.tiles_n = (g.N / 2 + gemm::BN / 2 - 1) / (gemm::BN / 2);
    a.b_half_rows = g.N / 2;
  } else {
    a.tiles_n = (g.N + gemm::BN - 1) / gemm::BN;
  }
  a.err = g.err;
#ifdef UCCL_EXPERIMENTS
  {
    const char* dbg = getenv("UCCL_FUSED_DEBUG");
    a.debug = dbg ? atoi(dbg) : 0;
  }
#endif
  // UCCL_GEMM_TIMES=1: CTA 0 stamps the phases of every launch; the launcher waits and prints them
  static unsigned long long* timesDev = nullptr;
#ifdef UCCL_EXPERIMENTS
  const bool wantTimes = getenv("UCCL_GEMM_TIMES") != nullptr;
#else
  const bool wantTimes = false;
#endif
  if (wantTimes) {
    if (!timesDev) cudaMalloc(&timesDev, 48 * sizeof(unsigned long long));
    cudaMemsetAsync(timesDev, 0, 48 * sizeof(unsigned long long), stream);
    a.times = timesDev;
  }
  const int sms = g.max_ctas > 0 ? g.max_ctas : deviceSmCount();
  gemm::PeerMaps pm = {};
  int comm_ctas = 0;
  if (role != 0) {
    if (f->nranks > gemm::kMaxPeers || f->rows_per_rank % gemm::BM != 0) return ucclInvalidArgument;
    gemm::CommArgs& c = a.comm;
    c.rank = f->rank;
    c.nranks = f->nranks;
    c.timeout_ns = f->timeout_ns;
    c.abort_flag = f->abort_flag;
    c.rows_per_rank = f->rows_per_rank;
    if (f->go && f->arena_peer && f->epochs) {
      // the fused kernels' own barrier slot: the last CTA index a collective may use
      constexpr int kSlot = kMaxBlocks - 1;
      for (int i = 0; i < f->nranks; ++i)
        c.bar_row_peer[i] = reinterpret_cast<uint32_t*>(f->arena_peer[i] + kArenaBarrierOff) + kSlot * kBarrierSlotWords;
      c.bar_epoch = f->epochs + kSlot;
      c.go = f->go;
    }
    const int blk_per_rank = f->rows_per_rank / gemm::BM;
    a.m_bpr = blk_per_rank;
    if (role == gemm::kCommAllGather) {
      comm_ctas = (f->a_external || f->a_spread) ? 0 : std::max(1, std::min(f->comm_ctas > 0 ? f->comm_ctas : 8, sms / 4));
      for (int i = 0; i < f->nranks; ++i) {
        c.a_full_peer[i] = static_cast<char*>(f->a_full_peer[i]);
        c.ready_peer[i] = f->ready_peer[i];
      }
      c.a_shard = static_cast<const char*>(f->a_shard);
      c.a_inplace = f->a_inplace;
      a.a_ready = f->ready_peer[f->rank];
      // one count per copied piece of a row block (see comm_allgather_push / _push2d)
      const size_t blkBytes = static_cast<size_t>(gemm::BM) * g.K * 2;
      a.a_spread = (!f->a_external && f->a_spread) ? 1 : 0;
      if (f->a_external) a.a_ready_target = 1;
      else if (a.a_spread) a.a_ready_target = static_cast<uint32_t>((blkBytes + gemm::FWD_SLOT_BYTES - 1) / gemm::FWD_SLOT_BYTES);
      else a.a_ready_target = static_cast<uint32_t>((blkBytes + gemm::COPY_SLOT_BYTES - 1) / gemm::COPY_SLOT_BYTES);
      a.a_local_lo = f->rank * blk_per_rank;
      a.a_local_hi = a.a_local_lo + blk_per_rank;
      if (!f->a_inplace) {
        // my rows are read straight from the shard; they reach A_full last, unobserved
        a.a_own_shard = 1;
        if (!makeTensorMap(&pm.m[0], f->a_shard, f->rows_per_rank, g.K, g.K, gemm::BK, gemm::BM)) return ucclSystemError;
      }
      a.m_order = (a.debug & 4) ? 0 : (f->a_peer_major ? 3 : 1);  // debug is zero outside experiment builds
    } else {
      for (int i = 0; i < f->nranks; ++i) {
        c.done_peer[i] = f->done_peer[i];
        // every rank's staging buffer is [nranks * rows_per_rank, N]: slot-major rows
        if (!makeTensorMap(&pm.m[i], f->stage_peer[i], static_cast<uint64_t>(f->nranks) * f->rows_per_rank, g.N, g.N, 64, 32))
          return ucclSystemError;
      }
      c.stage_local = static_cast<const char*>(f->stage_peer[f->rank]);
      c.done_target = static_cast<uint32_t>(f->nranks * a.tiles_n);
      c.rs_out = static_cast<char*>(f->rs_out);
      c.rs_ldo = f->rs_ldo;
      c.tail_next = f->tail_next;
      a.m_order = (a.debug & 4) ? 0 : 2;
    }
  }
  a.comm_ctas = comm_ctas;

  // Epilogue through shared memory + TMA stores: whole 128-byte lines instead of one 16-byte piece
  // per lane and row.  Needs 64-column boxes to tile the output exactly; the unicast forwarder warp
  // of the all-gather fusion uses the same staging area, so that mode keeps the direct stores.
  // (Experiment builds: UCCL_GEMM_EPI=lsu keeps the direct stores.)
  {
    const int outN = g.epilogue == gemm::kEpiSwiGLU ? g.N / 2 : g.N;
    bool tma = outN % 64 == 0 && role != gemm::kCommReduceScatter && !a.a_spread;
#ifdef UCCL_EXPERIMENTS
    if (const char* e = getenv("UCCL_GEMM_EPI")) {
      if (!strcasecmp(e, "lsu")) tma = false;
    }
#endif
    if (tma) {
      if (!makeTensorMap(&pm.m[gemm::kMaxPeers], g.C, g.M, outN, g.ldc, 64, 32)) return ucclSystemError;
      a.epi_tma = 1;
    }
  }

  const bool fusedOk = role == 0 || (f->rows_per_rank % (2 * gemm::BM) == 0);
  cudaError_t e;
  if (usePairKernel() && fusedOk) {
    // CTA pairs: 256-row tiles; both parts of the grid are even, and every cluster of the grid
    // must be resident at once because the GEMM CTAs of a fused launch wait for the
    // communication CTAs of the same launch
    const int tiles_m2 = (g.M + 2 * gemm::BM - 1) / (2 * gemm::BM);
    const int tiles2 = tiles_m2 * a.tiles_n;
    if (comm_ctas & 1) ++comm_ctas;
    a.comm_ctas = comm_ctas;
    int maxPairs = maxResidentPairs();
    if (g.max_ctas > 0) maxPairs = std::min(maxPairs, g.max_ctas / 2);
    // reducer CTAs (reduce-scatter only, and only with the shared work counter) come out of the
    // resident budget: they must run from the start, next to the GEMM CTAs
    int reducers = 0;
    if (role == gemm::kCommReduceScatter && f->tail_next && f->rs_reducers > 0)
      reducers = std::min(f->rs_reducers & ~1, maxPairs & ~1);  // whole clusters, at most half of the resident CTAs
    int pairs = std::max(1, std::min(maxPairs - comm_ctas / 2 - reducers / 2, tiles2));
    a.gemm_ctas = 2 * pairs;
    const int grid = a.gemm_ctas + comm_ctas + reducers;
    if (g.epilogue == gemm::kEpiSwiGLU) {
      if (role == gemm::kCommAllGather) e = launchPairT<gemm::kEpiSwiGLU, gemm::kCommAllGather>(tmA, tmB, pm, a, grid, stream);
      else e = launchPairT<gemm::kEpiSwiGLU, gemm::kCommNone>(tmA, tmB, pm, a, grid, stream);
    } else {
      if (role == gemm::kCommAllGather) e = launchPairT<gemm::kEpiStore, gemm::kCommAllGather>(tmA, tmB, pm, a, grid, stream);
      else if (role == gemm::kCommReduceScatter) e = launchPairT<gemm::kEpiStore, gemm::kCommReduceScatter>(tmA, tmB, pm, a, grid, stream);
      else e = launchPairT<gemm::kEpiStore, gemm::kCommNone>(tmA, tmB, pm, a, grid, stream);
    }
  } else {
    const int tiles = a.tiles_m * a.tiles_n;
    int reducers = 0;
    if (role == gemm::kCommReduceScatter && f->tail_next && f->rs_reducers > 0) reducers = std::min(f->rs_reducers, sms / 2);
    a.gemm_ctas = std::max(1, std::min(sms - comm_ctas - reducers, tiles));
    const int grid = a.gemm_ctas + comm_ctas + reducers;
    if (g.epilogue == gemm::kEpiSwiGLU) {
      if (role == gemm::kCommAllGather) e = launchT<gemm::kEpiSwiGLU, gemm::kCommAllGather>(tmA, tmB, pm, a, grid, stream);
      else e = launchT<gemm::kEpiSwiGLU, gemm::kCommNone>(tmA, tmB, pm, a, grid, stream);
    } else {
      if (role == gemm::kCommAllGather) e = launchT<gemm::kEpiStore, gemm::kCommAllGather>(tmA, tmB, pm, a, grid, stream);
      else if (role == gemm::kCommReduceScatter) e = launchT<gemm::kEpiStore, gemm::kCommReduceScatter>(tmA, tmB, pm, a, grid, stream);
      else e = launchT<gemm::kEpiStore, gemm::kCommNone>(tmA, tmB, pm, a, grid, stream);
    }
  }
  if (e != cudaSuccess) {
    UCCL_LOG(ERROR, "gemm launch failed: %s", cudaGetErrorString(e));
    return ucclSystemError;
  }
  if (wantTimes && cudaStreamSynchronize(stream) == cudaSuccess) {
    unsigned long long t[48];
    cudaMemcpy(t, timesDev, sizeof(t), cudaMemcpyDeviceToHost);
    fprintf(stderr, "[gemm times] role %d: main loop %.1f us, tail setup %.1f us, units:", role,
            t[1] > t[0] ? (t[1] - t[0]) * 1e-3 : 0.0, t[2] > t[1] ? (t[2] - t[1]) * 1e-3 : 0.0);
    for (int i = 3; i < 15 && t[i]; ++i) fprintf(stderr, " %.1f", (t[i] - t[i - 1]) * 1e-3);
    fprintf(stderr, " | wait/sum:");
    for (int i = 0; i < 8 && t[16 + 2 * i]; ++i)
      fprintf(stderr, " %.1f/%.1f", (t[16 + 2 * i] - t[2]) * 1e-3, (t[17 + 2 * i] - t[16 + 2 * i]) * 1e-3);
    fprintf(stderr, "\n");
  }
  return ucclSuccess;
}

}  // namespace uccl

extern "C" ucclResult_t ucclGemmBf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                     int ldc, int epilogue, void* stream) {
  uccl::GemmLaunch g;
  g.A = A;
  g.B = B;
  g.C = C;
  g.M = M;
  g.N = N;
  g.K = K;
  g.lda = lda;
  g.ldb = ldb;
  g.ldc = ldc;
  g.epilogue = epilogue;
  return uccl::launchGemmBf16(g, nullptr, static_cast<cudaStream_t>(stream));
}
