// Allocation-free single-GPU MoE dispatch (see include/uccl_noalloc.h for the contract).
//
// The scratch memory that the regular dispatch kernel gets from its context object is a
// file-scope device array here.  In host code the name of that array is only a stand-in for the
// symbol -- it is not a device address -- so the address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and that pointer is what the kernel receives.
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include <mutex>

#include "ptx.cuh"
#include "uccl_noalloc.h"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxIter = 32;  // 256 elements per warp iteration -> hidden <= 8192
constexpr int kMaxDevices = 64;

// [0, 4)   rows claimed so far      [4, 8) CTAs finished      [8, 12) rows dropped
// [1024, ...) row slot of every (token, k) pair, int32
static __device__ __align__(256) unsigned char g_noalloc_scratch[UCCL_NOALLOC_SCRATCH_BYTES];

struct Scratch {
  unsigned int* rows;
  unsigned int* ctasDone;
  unsigned int* dropped;
  int* slotOf;
};

__global__ void __launch_bounds__(kThreads) moe_dispatch_local_kernel(unsigned char* scratch, const void* x,
                                                                      const int32_t* topkIdx, int tokens, int H, int topk,
                                                                      int numExperts, char* recvX, float* recvScale,
                                                                      int32_t* recvMeta, int32_t* recvCount,
                                                                      int rowsCapacity) {
  using namespace uccl;
  Scratch sc;
  sc.rows = reinterpret_cast<unsigned int*>(scratch);
  sc.ctasDone = sc.rows + 1;
  sc.dropped = sc.rows + 2;
  sc.slotOf = reinterpret_cast<int*>(scratch + 1024);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warpsPerCta = kThreads / 32;
  const int nblk = H / 128, iters = (H + 255) / 256, half = lane >> 4;

  for (int t = blockIdx.x * warpsPerCta + warp; t < tokens; t += gridDim.x * warpsPerCta) {
    const char* row = static_cast<const char*>(x) + static_cast<size_t>(t) * H * 2;
    uint2 q[kMaxIter];
    float scaleLo = 0.f, scaleHi = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxIter; ++i) {
      if (i < iters) {
        const bool live = 2 * i + half < nblk;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (live) v = ptx::ld_global_v4(row + (static_cast<size_t>(i) * 256 + lane * 8) * 2);
        float f[8];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 p = ptx::unpack_bf16x2(w[j]);
          f[2 * j] = p.x;
          f[2 * j + 1] = p.y;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float scale = fmaxf(amax, 1e-10f) / 448.f;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const __nv_fp8x2_storage_t a0 = __nv_cvt_float2_to_fp8x2(
              make_float2(__fdiv_rn(f[4 * j], scale), __fdiv_rn(f[4 * j + 1], scale)), __NV_SATFINITE, __NV_E4M3);
          const __nv_fp8x2_storage_t a1 = __nv_cvt_float2_to_fp8x2(
              make_float2(__fdiv_rn(f[4 * j + 2], scale), __fdiv_rn(f[4 * j + 3], scale)), __NV_SATFINITE, __NV_E4M3);
          const uint32_t word = static_cast<uint32_t>(a0) | (static_cast<uint32_t>(a1) << 16);
          if (j == 0) lo = word; else hi = word;
        }
        q[i] = make_uint2(lo, hi);
        const float s = __shfl_sync(0xffffffffu, scale, (lane & 1) * 16);
        if ((lane >> 1) == (i & 15)) {
          if (i < 16) scaleLo = s; else scaleHi = s;
        }
      }
    }
    for (int k = 0; k < topk; ++k) {
      const int e = topkIdx[static_cast<size_t>(t) * topk + k];
      int slot = -1;
      if (e >= 0 && e < numExperts) {
        if (lane == 0) slot = static_cast<int>(atomicAdd(sc.rows, 1u));
        slot = __shfl_sync(0xffffffffu, slot, 0);
        if (slot >= rowsCapacity) {
          if (lane == 0) atomicAdd(sc.dropped, 1u);
          slot = -1;
        }
      }
      if (lane == 0) sc.slotOf[static_cast<size_t>(t) * topk + k] = slot;
      if (slot < 0) continue;
      char* xdst = recvX + static_cast<size_t>(slot) * H;
#pragma unroll
      for (int i = 0; i < kMaxIter; ++i)
        if (i < iters && 2 * i + half < nblk)
          *reinterpret_cast<uint2*>(xdst + static_cast<size_t>(i) * 256 + lane * 8) = q[i];
      float* sdst = recvScale + static_cast<size_t>(slot) * nblk;
      if (lane < nblk) sdst[lane] = scaleLo;
      if (32 + lane < nblk) sdst[32 + lane] = scaleHi;
      if (lane == 0) *reinterpret_cast<int4*>(recvMeta + static_cast<size_t>(slot) * 4) = make_int4(t, e, k, 1);
    }
  }
  // the last CTA to finish publishes the row count
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = atomicAdd(sc.ctasDone, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    __threadfence();
    const unsigned int rows = *reinterpret_cast<volatile unsigned int*>(sc.rows);
    *recvCount = static_cast<int32_t>(rows < static_cast<unsigned int>(rowsCapacity) ? rows : rowsCapacity);
  }
}

thread_local char t_err[256] = "";
ucclResult_t refuse(ucclResult_t r, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return r;
}

// Device address of the scratch array, looked up once per device (with that device current).
unsigned char* g_scratchPtr[kMaxDevices];
std::mutex g_setupMu;

ucclResult_t scratchForCurrentDevice(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return refuse(ucclSystemError, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return refuse(ucclInvalidArgument, "device index %d is out of range", dev);
  std::lock_guard<std::mutex> lk(g_setupMu);
  if (!g_scratchPtr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return refuse(ucclSystemError, "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    }
    g_scratchPtr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratchPtr[dev];
  return ucclSuccess;
}

}  // namespace

extern "C" ucclResult_t ucclMoeDispatchLocalNoAlloc(const void* x, const int32_t* topkIdx, int tokens, int hidden,
                                                    int numExperts, int topk, void* recvX, float* recvScale,
                                                    int32_t* recvMeta, int32_t* recvCount, int rowsCapacity,
                                                    void* stream) {
  t_err[0] = 0;
  if (!x || !topkIdx || !recvX || !recvScale || !recvMeta || !recvCount)
    return refuse(ucclInvalidArgument, "null buffer");
  if (tokens < 0 || tokens > UCCL_NOALLOC_MAX_TOKENS)
    return refuse(ucclInvalidArgument, "tokens = %d exceeds the built-in scratch (at most %d)", tokens, UCCL_NOALLOC_MAX_TOKENS);
  if (topk < 1 || topk > UCCL_NOALLOC_MAX_TOPK)
    return refuse(ucclInvalidArgument, "topk = %d exceeds the built-in scratch (1..%d)", topk, UCCL_NOALLOC_MAX_TOPK);
  if (hidden <= 0 || hidden % 128 != 0 || hidden > kMaxIter * 256)
    return refuse(ucclInvalidArgument, "hidden = %d must be a multiple of 128 and at most %d", hidden, kMaxIter * 256);
  if (numExperts < 1) return refuse(ucclInvalidArgument, "numExperts must be positive");
  if (static_cast<long>(rowsCapacity) < static_cast<long>(tokens) * topk)
    return refuse(ucclInvalidArgument, "rowsCapacity = %d is smaller than tokens * topk = %ld", rowsCapacity,
                  static_cast<long>(tokens) * topk);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(recvX) | reinterpret_cast<uintptr_t>(recvMeta)) & 15)
    return refuse(ucclInvalidArgument, "x, recvX and recvMeta must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(recvScale) | reinterpret_cast<uintptr_t>(topkIdx) | reinterpret_cast<uintptr_t>(recvCount)) & 3)
    return refuse(ucclInvalidArgument, "recvScale, topkIdx and recvCount must be 4-byte aligned");
  unsigned char* scratch = nullptr;
  ucclResult_t r = scratchForCurrentDevice(&scratch);
  if (r != ucclSuccess) return r;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: the three counters must start at zero
  cudaError_t e = cudaMemsetAsync(scratch, 0, 16, s);
  if (e != cudaSuccess) return refuse(ucclSystemError, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  if (tokens == 0) {
    e = cudaMemsetAsync(recvCount, 0, sizeof(int32_t), s);
    return e == cudaSuccess ? ucclSuccess : refuse(ucclSystemError, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  }
  int ctas = (tokens + 7) / 8;
  ctas = ctas > 592 ? 592 : ctas;
  moe_dispatch_local_kernel<<<ctas, kThreads, 0, s>>>(scratch, x, topkIdx, tokens, hidden, topk, numExperts,
                                                      static_cast<char*>(recvX), recvScale, recvMeta, recvCount,
                                                      rowsCapacity);
  e = cudaGetLastError();
  if (e != cudaSuccess) return refuse(ucclSystemError, "kernel launch failed: %s", cudaGetErrorString(e));
  return ucclSuccess;
}

extern "C" const char* ucclNoAllocLastError(void) { return t_err; }
