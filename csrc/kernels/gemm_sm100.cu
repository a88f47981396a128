// Launchers for the tcgen05 GEMM: tensor-map construction, grid sizing, template dispatch.
#include "gemm_sm100.h"

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
  int gemm_ctas = sms - comm_ctas;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  a.gemm_ctas = gemm_ctas;
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
