// MoE expert-parallel dispatch and combine as single kernels over NVLink peer memory.
//
// dispatch : one warp per token.  The warp reads the bf16 row once, computes an fp32 scale per
//            128 elements (amax / 448), converts to fp8 e4m3 and keeps the converted row in
//            registers; for every selected expert it takes a row slot in the region this rank owns
//            on the expert's rank (local atomic: no cross-rank contention) and stores the fp8
//            row, the scales and a 16-byte descriptor {token, local expert, k, 1} straight into
//            that rank's receive area.  The last CTA publishes the per-destination row counts and
//            raises an arrival flag on every rank, then waits for everybody else's flag, so the
//            receive area is complete when the kernel ends.
// combine  : one warp per token pulls the bf16 expert outputs of its top-k rows from the ranks
//            that computed them (eight 16-byte loads in flight per lane), multiplies by the
//            routing weights, accumulates in fp32 and writes the bf16 result.
// Neither exists in the reference (it has no all-to-all at all, desgin/design-spec.md:1760).
#include <cuda_fp8.h>

#include "coll_device.cuh"
#include "moe.h"

namespace uccl {
namespace dev {

constexpr int kMoeThreads = 256;
constexpr int kMoeMaxIter = 32;   // 256 elements per warp iteration -> hidden <= 8192
constexpr int kMoeMaxTopk = 16;

__global__ void __launch_bounds__(kMoeThreads) moe_dispatch_kernel(const __grid_constant__ MoeArgs a) {
  const DevComm& dc = a.dc;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warpsPerCta = kMoeThreads / 32;
  const int n = dc.nranks, me = dc.rank;
  const int H = a.hidden, nblk = H / 128;
  const int iters = (H + 255) / 256;
  const int half = lane >> 4;  // which of the two 128-element blocks of an iteration

  for (int t = blockIdx.x * warpsPerCta + warp; t < a.tokens; t += gridDim.x * warpsPerCta) {
    const char* row = static_cast<const char*>(a.x) + static_cast<size_t>(t) * H * 2;
    uint2 q[kMoeMaxIter];
    float scaleLo = 0.f, scaleHi = 0.f;  // lane l ends up with the scales of blocks l and 32 + l
    // the row is read in batches of eight 16-byte loads per lane, all issued before the first use
    constexpr int kBatch = 8;
    uint4 vb[kBatch];
#pragma unroll
    for (int i = 0; i < kMoeMaxIter; ++i) {
      if ((i % kBatch) == 0) {
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          vb[j] = make_uint4(0, 0, 0, 0);
          if (i + j < iters && 2 * (i + j) + half < nblk)
            vb[j] = ptx::ld_global_v4(row + (static_cast<size_t>(i + j) * 256 + lane * 8) * 2);
        }
      }
      if (i < iters) {
        const uint4 v = vb[i % kBatch];
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
        // x / scale with a true division: bit-identical to the fp32 restatement of the cast, so
        // no element lands on the other side of an fp8 rounding boundary
        const float scale = fmaxf(amax, 1e-10f) / 448.f;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const __nv_fp8x2_storage_t a0 = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(f[4 * j], scale), __fdiv_rn(f[4 * j + 1], scale)), __NV_SATFINITE, __NV_E4M3);
          const __nv_fp8x2_storage_t a1 = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(f[4 * j + 2], scale), __fdiv_rn(f[4 * j + 3], scale)), __NV_SATFINITE, __NV_E4M3);
          const uint32_t word = static_cast<uint32_t>(a0) | (static_cast<uint32_t>(a1) << 16);
          if (j == 0) lo = word; else hi = word;
        }
        q[i] = make_uint2(lo, hi);
        // hand the scale of block (2i + h) to lane (2i + h) mod 32
        const float s = __shfl_sync(0xffffffffu, scale, (lane & 1) * 16);
        if ((lane >> 1) == (i & 15)) {
          if (i < 16) scaleLo = s; else scaleHi = s;
        }
      }
    }
    // routing
    for (int k = 0; k < a.topk; ++k) {
      const int e = a.topkIdx[static_cast<size_t>(t) * a.topk + k];
      int slot = -1, dst = 0;
      if (e >= 0 && e < a.numExperts) {
        dst = e / a.expertsPerRank;
        if (lane == 0) slot = static_cast<int>(atomicAdd(a.sendCount + dst, 1u));
        slot = __shfl_sync(0xffffffffu, slot, 0);
        if (slot >= a.rowsPerSource) {
          if (lane == 0) atomicAdd(a.overflow, 1u);
          slot = -1;
        }
      }
      if (lane == 0) a.slotOf[static_cast<size_t>(t) * a.topk + k] = slot < 0 ? -1 : ((dst << 24) | slot);
      if (slot < 0) continue;
      const size_t r = static_cast<size_t>(me) * a.rowsPerSource + slot;
      char* xdst = a.recvX[dst] + r * H;
#pragma unroll
      for (int i = 0; i < kMoeMaxIter; ++i)
        if (i < iters && 2 * i + half < nblk)
          *reinterpret_cast<uint2*>(xdst + static_cast<size_t>(i) * 256 + lane * 8) = q[i];
      float* sdst = a.recvScale[dst] + r * nblk;
      if (lane < nblk) sdst[lane] = scaleLo;
      if (32 + lane < nblk) sdst[32 + lane] = scaleHi;
      if (lane == 0)
        *reinterpret_cast<int4*>(a.recvMeta[dst] + r * 4) = make_int4(t, e - dst * a.expertsPerRank, k, 1);
    }
  }

  // ---- completion: the last CTA publishes counts and flags, then waits for every source
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    ptx::fence_sys();
    const uint32_t prev = atomicAdd(a.ctasDone, 1u);
    s_last = prev == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const uint32_t e = *a.epoch + 1;
  if (threadIdx.x < static_cast<unsigned>(n)) {
    const int p = threadIdx.x;
    const uint32_t cnt = min(*reinterpret_cast<volatile uint32_t*>(a.sendCount + p), static_cast<uint32_t>(a.rowsPerSource));
    a.recvCounts[p][me] = static_cast<int32_t>(cnt);
    ptx::fence_sys();
    ptx::st_release_sys_u32(a.arrived[p] + me, e);
  }
  __syncthreads();
  if (threadIdx.x < static_cast<unsigned>(n)) {
    a.sendCount[threadIdx.x] = 0;  // ready for the next call
    wait_u32(a.arrived[me] + threadIdx.x, e, dc, DEV_TIMEOUT_MOE, threadIdx.x, e);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *a.ctasDone = 0;
    *a.epoch = e;
  }
}

__global__ void __launch_bounds__(kMoeThreads) moe_combine_kernel(const __grid_constant__ MoeArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warpsPerCta = kMoeThreads / 32;
  const int me = a.dc.rank, H = a.hidden;
  const int iters = (H + 255) / 256;
  for (int t = blockIdx.x * warpsPerCta + warp; t < a.tokens; t += gridDim.x * warpsPerCta) {
    const char* src[kMoeMaxTopk];
    float w[kMoeMaxTopk];
#pragma unroll
    for (int k = 0; k < kMoeMaxTopk; ++k) {
      src[k] = nullptr;
      w[k] = 0.f;
      if (k < a.topk) {
        const int s = a.slotOf[static_cast<size_t>(t) * a.topk + k];
        if (s >= 0) {
          const int dst = s >> 24, slot = s & 0xffffff;
          src[k] = a.expertOut[dst] + (static_cast<size_t>(me) * a.rowsPerSource + slot) * H * 2;
          w[k] = a.topkWeight[static_cast<size_t>(t) * a.topk + k];
        }
      }
    }
    char* orow = static_cast<char*>(a.out) + static_cast<size_t>(t) * H * 2;
    for (int i = 0; i < iters; ++i) {
      const size_t off = (static_cast<size_t>(i) * 256 + lane * 8) * 2;
      if (i * 256 + lane * 8 >= H) continue;
      uint4 v[kMoeMaxTopk];
#pragma unroll
      for (int k = 0; k < kMoeMaxTopk; ++k)
        if (k < a.topk && src[k]) v[k] = ptx::ld_stream_v4(src[k] + off);
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int k = 0; k < kMoeMaxTopk; ++k) {
        if (k < a.topk && src[k]) {
          const uint32_t u[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 p = ptx::unpack_bf16x2(u[j]);
            acc[2 * j] += w[k] * p.x;
            acc[2 * j + 1] += w[k] * p.y;
          }
        }
      }
      ptx::st_global_v4(orow + off, Vec<DT_BF16>::pack(acc));
    }
  }
}

}  // namespace dev

cudaError_t launchMoeDispatch(const MoeArgs& a, cudaStream_t stream) {
  if (a.hidden % 128 != 0 || a.hidden > dev::kMoeMaxIter * 256 || a.topk < 1 || a.topk > dev::kMoeMaxTopk)
    return cudaErrorInvalidValue;
  int ctas = (a.tokens + 7) / 8;
  ctas = ctas < 1 ? 1 : (ctas > 592 ? 592 : ctas);
  dev::moe_dispatch_kernel<<<ctas, dev::kMoeThreads, 0, stream>>>(a);
  return cudaGetLastError();
}
cudaError_t launchMoeCombine(const MoeArgs& a, cudaStream_t stream) {
  if (a.hidden % 128 != 0 || a.hidden > dev::kMoeMaxIter * 256 || a.topk < 1 || a.topk > dev::kMoeMaxTopk)
    return cudaErrorInvalidValue;
  int ctas = (a.tokens + 7) / 8;
  ctas = ctas < 1 ? 1 : (ctas > 592 ? 592 : ctas);
  dev::moe_combine_kernel<<<ctas, dev::kMoeThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace uccl
