// Launchers for the tcgen05 GEMM: tensor-map construction, grid sizing, template dispatch.
#include "gemm_sm100.h"

#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include <mutex>

#include "../core/cuda_driver.h"
#include "../core/log.h"
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

// K-major bf16 matrix [rows, cols] with 128-byte swizzled 64-column boxes.
bool makeTensorMap(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                   uint32_t box_rows) {
  const DriverApi& d = driverApi();
  if (!d.ok) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(gemm::BK), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = d.tensorMapEncodeTiled(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                                      dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    UCCL_LOG(ERROR, "cuTensorMapEncodeTiled failed: %s (base=%p rows=%llu cols=%llu ld=%llu)",
             driverErrorString(r), base, (unsigned long long)rows, (unsigned long long)cols,
             (unsigned long long)ld);
    return false;
  }
  return true;
}

template <int EPI, int COMM>
cudaError_t launchT(const CUtensorMap& tmA, const CUtensorMap& tmB, const gemm::Args& args, int grid,
                    cudaStream_t stream) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  auto kern = gemm::gemm_bf16_kernel<EPI, COMM>;
  // The attribute is per device; setting it again is cheap, so do it on every device switch.
  static thread_local int last_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != last_dev) {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::SMEM_BYTES);
    last_dev = dev;
  }
  (void)once;
  if (attr_err != cudaSuccess) return attr_err;
  kern<<<grid, gemm::NUM_THREADS, gemm::SMEM_BYTES, stream>>>(tmA, tmB, args);
  return cudaGetLastError();
}

template <int EPI, int COMM>
cudaError_t launchPairT(const CUtensorMap& tmA, const CUtensorMap& tmB, const gemm::Args& args, int grid,
                        cudaStream_t stream) {
  auto kern = gemm::gemm2_bf16_kernel<EPI, COMM>;
  static thread_local int last_dev = -1;
  static cudaError_t attr_err = cudaSuccess;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != last_dev) {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::pair::SMEM_BYTES);
    last_dev = dev;
  }
  if (attr_err != cudaSuccess) return attr_err;
  kern<<<grid, gemm::NUM_THREADS, gemm::pair::SMEM_BYTES, stream>>>(tmA, tmB, args);
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
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm::pair::SMEM_BYTES);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * deviceSmCount(), 1, 1);
    cfg.blockDim = dim3(gemm::NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = gemm::pair::SMEM_BYTES;
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
  static int v = -1;
  if (v < 0) {
    const char* s = getenv("UCCL_GEMM_PAIR");
    v = (s && *s) ? (atoi(s) != 0) : 1;
  }
  return v != 0;
}

}  // namespace

ucclResult_t launchGemmBf16(const GemmLaunch& g, const GemmFusion* f, cudaStream_t stream) {
  if (!g.A || !g.B || !g.C || g.M <= 0 || g.N <= 0 || g.K <= 0) return ucclInvalidArgument;
  if (g.K % 8 != 0 || g.lda % 8 != 0 || g.ldb % 8 != 0 || g.ldc % 8 != 0) return ucclInvalidArgument;
  if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B) |
       reinterpret_cast<uintptr_t>(g.C)) & 15)
    return ucclInvalidArgument;
  if (g.epilogue == gemm::kEpiSwiGLU && (g.N % 2 != 0)) return ucclInvalidArgument;

  CUtensorMap tmA, tmB;
  if (!makeTensorMap(&tmA, g.A, g.M, g.K, g.lda, gemm::BM)) return ucclSystemError;
  if (!makeTensorMap(&tmB, g.B, g.N, g.K, g.ldb, gemm::BN / 2)) return ucclSystemError;

  gemm::Args a{};
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
  const int sms = g.max_ctas > 0 ? g.max_ctas : deviceSmCount();
  const int tiles = a.tiles_m * a.tiles_n;
  int role = f ? f->role : 0;
  int comm_ctas = 0;
  if (role != 0) {
    comm_ctas = f->comm_ctas > 0 ? f->comm_ctas : 8;
    if (comm_ctas > sms / 2) comm_ctas = sms / 2;
    gemm::CommArgs& c = a.comm;
    c.rank = f->rank;
    c.nranks = f->nranks;
    c.use_multimem = f->use_multimem;
    c.epoch = f->epoch;
    c.timeout_ns = f->timeout_ns;
    c.abort_flag = f->abort_flag;
    c.rows_per_rank = f->rows_per_rank;
    c.a_local = f->a_local;
    c.a_full_mc = f->a_full_mc;
    c.c_part_mc = f->c_part_mc;
    c.rs_out = f->rs_out;
    c.rs_ldo = f->rs_ldo;
    for (int i = 0; i < f->nranks && i < gemm::kMaxPeers; ++i) {
      c.a_full_peer[i] = f->a_full_peer[i];
      c.ready_peer[i] = f->ready_peer[i];
      c.c_part_peer[i] = f->c_part_peer[i];
      c.done_peer[i] = f->done_peer[i];
    }
    if (f->rows_per_rank % gemm::BM != 0) return ucclInvalidArgument;
    const int blk_per_rank = f->rows_per_rank / gemm::BM;
    if (role == gemm::kCommAllGatherPush) {
      a.a_ready = f->ready_peer[f->rank];
      a.a_ready_target = f->epoch;
      // the local shard is copied into A_full by the communication CTAs as well, so its rows
      // are awaited like everybody else's; they simply arrive first
      a.a_local_lo = a.a_local_hi = 0;
      a.m_order = 1;
      a.m_bpr = blk_per_rank;
    } else {
      a.m_order = 2;
      a.m_bpr = blk_per_rank;
    }
  }
  const bool fusedOk = role == 0 || (f->rows_per_rank % (2 * gemm::BM) == 0);
  if (usePairKernel() && fusedOk) {
    // CTA pairs: 256-row tiles, both the GEMM part and the communication part of the grid are even
    const int tiles_m2 = (g.M + 2 * gemm::BM - 1) / (2 * gemm::BM);
    const int tiles2 = tiles_m2 * a.tiles_n;
    if (comm_ctas & 1) ++comm_ctas;
    // every cluster of the grid must be resident at once: the GEMM CTAs of a fused launch wait
    // for the communication CTAs of the same launch
    int maxPairs = maxResidentPairs();
    if (g.max_ctas > 0) maxPairs = std::min(maxPairs, g.max_ctas / 2);
    int pairs = maxPairs - comm_ctas / 2;
    if (pairs > tiles2) pairs = tiles2;
    if (pairs < 1) pairs = 1;
    a.gemm_ctas = 2 * pairs;
    a.comm_ctas = comm_ctas;
    const int grid2 = a.gemm_ctas + comm_ctas;
    cudaError_t e2;
    if (g.epilogue == gemm::kEpiSwiGLU) {
      if (role == gemm::kCommAllGatherPush) e2 = launchPairT<gemm::kEpiSwiGLU, gemm::kCommAllGatherPush>(tmA, tmB, a, grid2, stream);
      else if (role == 0) e2 = launchPairT<gemm::kEpiSwiGLU, gemm::kCommNone>(tmA, tmB, a, grid2, stream);
      else return ucclInvalidArgument;
    } else {
      if (role == gemm::kCommAllGatherPush) e2 = launchPairT<gemm::kEpiStore, gemm::kCommAllGatherPush>(tmA, tmB, a, grid2, stream);
      else if (role == gemm::kCommReduceScatter) e2 = launchPairT<gemm::kEpiStore, gemm::kCommReduceScatter>(tmA, tmB, a, grid2, stream);
      else e2 = launchPairT<gemm::kEpiStore, gemm::kCommNone>(tmA, tmB, a, grid2, stream);
    }
    if (e2 != cudaSuccess) {
      UCCL_LOG(ERROR, "gemm (CTA pair) launch failed: %s", cudaGetErrorString(e2));
      return ucclSystemError;
    }
    return ucclSuccess;
  }

  int gemm_ctas = sms - comm_ctas;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  a.gemm_ctas = gemm_ctas;
  a.comm_ctas = comm_ctas;
  const int grid = gemm_ctas + comm_ctas;

  cudaError_t e;
  if (g.epilogue == gemm::kEpiSwiGLU) {
    if (role == gemm::kCommAllGatherPush)
      e = launchT<gemm::kEpiSwiGLU, gemm::kCommAllGatherPush>(tmA, tmB, a, grid, stream);
    else if (role == 0)
      e = launchT<gemm::kEpiSwiGLU, gemm::kCommNone>(tmA, tmB, a, grid, stream);
    else
      return ucclInvalidArgument;
  } else {
    if (role == gemm::kCommAllGatherPush)
      e = launchT<gemm::kEpiStore, gemm::kCommAllGatherPush>(tmA, tmB, a, grid, stream);
    else if (role == gemm::kCommReduceScatter)
      e = launchT<gemm::kEpiStore, gemm::kCommReduceScatter>(tmA, tmB, a, grid, stream);
    else
      e = launchT<gemm::kEpiStore, gemm::kCommNone>(tmA, tmB, a, grid, stream);
  }
  if (e != cudaSuccess) {
    UCCL_LOG(ERROR, "gemm launch failed: %s", cudaGetErrorString(e));
    return ucclSystemError;
  }
  return ucclSuccess;
}

}  // namespace uccl

extern "C" ucclResult_t ucclGemmBf16(const void* A, const void* B, void* C, int M, int N, int K, int lda,
                                     int ldb, int ldc, int epilogue, void* stream) {
  uccl::GemmLaunch g;
  g.A = A; g.B = B; g.C = C;
  g.M = M; g.N = N; g.K = K;
  g.lda = lda; g.ldb = ldb; g.ldc = ldc;
  g.epilogue = epilogue;
  return uccl::launchGemmBf16(g, nullptr, static_cast<cudaStream_t>(stream));
}
