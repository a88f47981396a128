// MoE expert-parallel dispatch and combine as single kernels over NVLink peer memory.
//
// dispatch : one warp per token, in two steps.  Quantise: the warp reads the bf16 row once,
//            computes an fp32 scale per 128 elements (amax / 448), converts to fp8 e4m3 and writes
//            the converted row and its scales into the warp's slice of shared memory (nothing of
//            the row stays in registers, which is what lets three CTAs share an SM).  Scatter: lane
//            k takes a row slot for the token's k-th expert in the region this rank owns on the
//            expert's rank (local atomic: no cross-rank contention) and issues bulk copies
//            shared memory -> that rank's receive area for the row and the scales, plus a 16-byte
//            descriptor {token, local expert, k, 1}: the SM's copy engine moves the 7 KiB rows
//            while the warp already converts its next token.  The last CTA publishes the
//            per-destination row counts and raises an arrival flag on every rank, then waits for
//            everybody else's flag, so the receive area is complete when the kernel ends.
// combine  : one warp per token pulls the bf16 expert outputs of its top-k rows from the ranks
//            that computed them (sixteen 16-byte loads in flight per lane), multiplies by the
//            routing weights, accumulates in fp32 and writes the bf16 result.
// Neither exists in the reference (it has no all-to-all at all, desgin/design-spec.md:1760).
#include <cuda_fp8.h>

#include "coll_device.cuh"
#include "moe.h"

namespace uccl {
namespace dev {

constexpr int kMoeThreads = 256;
constexpr int kMoeMaxIter = 32;   // combine: 256 elements per warp iteration -> hidden <= 8192
constexpr int kMoeMaxTopk = 16;

// shared memory of one warp: the quantised row, then its scales
__host__ __device__ constexpr int moe_warp_smem(int hidden) { return hidden + ((hidden / 128 * 4 + 15) & ~15); }

__global__ void __launch_bounds__(kMoeThreads, 3) moe_dispatch_kernel(const __grid_constant__ MoeArgs a) {
  extern __shared__ __align__(16) uint8_t moe_smem[];
  const DevComm& dc = a.dc;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warpsPerCta = kMoeThreads / 32;
  const int n = dc.nranks, me = dc.rank;
  const int H = a.hidden, nblk = H / 128;
  const int iters = (H + 511) / 512;  // a lane converts 16 consecutive elements per iteration
  uint8_t* rowBuf = moe_smem + static_cast<size_t>(warp) * moe_warp_smem(H);
  float* scaleBuf = reinterpret_cast<float*>(rowBuf + H);
  const uint32_t scaleBytes = static_cast<uint32_t>(nblk) * 4;
  const bool scalesBulk = (scaleBytes & 15u) == 0;  // a bulk copy moves multiples of 16 bytes

  for (int t = blockIdx.x * warpsPerCta + warp; t < a.tokens; t += gridDim.x * warpsPerCta) {
    const char* row = static_cast<const char*>(a.x) + static_cast<size_t>(t) * H * 2;
    // the bulk copies of the previous token must have read the buffers before they are rewritten
    if (lane < a.topk) ptx::tma_store_wait_read<0>();
    __syncwarp();
    // ---- quantise: the row is read in batches of four iterations (eight 16-byte loads per lane
    // in flight), converted 16 elements at a time and written to shared memory as one 16-byte store
    constexpr int kBatch = 4;
    for (int i0 = 0; i0 < iters; i0 += kBatch) {
      uint4 v[kBatch][2];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int e0 = (i0 + j) * 512 + lane * 16;
        v[j][0] = v[j][1] = make_uint4(0, 0, 0, 0);
        if (i0 + j < iters && e0 < H) {
          v[j][0] = ptx::ld_global_v4(row + static_cast<size_t>(e0) * 2);
          v[j][1] = ptx::ld_global_v4(row + static_cast<size_t>(e0) * 2 + 16);
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (i0 + j >= iters) break;  // uniform over the warp
        const int e0 = (i0 + j) * 512 + lane * 16;
        float f[16];
        const uint32_t w[8] = {v[j][0].x, v[j][0].y, v[j][0].z, v[j][0].w, v[j][1].x, v[j][1].y, v[j][1].z, v[j][1].w};
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float2 p = ptx::unpack_bf16x2(w[q]);
          f[2 * q] = p.x;
          f[2 * q + 1] = p.y;
        }
        float amax = 0.f;
#pragma unroll
        for (int q = 0; q < 16; ++q) amax = fmaxf(amax, fabsf(f[q]));
        // a 128-element block is eight lanes
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        // x / scale with a true division: bit-identical to the fp32 restatement of the cast, so
        // no element lands on the other side of an fp8 rounding boundary
        const float scale = fmaxf(amax, 1e-10f) / 448.f;
        uint32_t o32[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const __nv_fp8x2_storage_t a0 = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(f[4 * q], scale), __fdiv_rn(f[4 * q + 1], scale)), __NV_SATFINITE, __NV_E4M3);
          const __nv_fp8x2_storage_t a1 = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(f[4 * q + 2], scale), __fdiv_rn(f[4 * q + 3], scale)), __NV_SATFINITE, __NV_E4M3);
          o32[q] = static_cast<uint32_t>(a0) | (static_cast<uint32_t>(a1) << 16);
        }
        if (e0 < H) {
          *reinterpret_cast<uint4*>(rowBuf + e0) = make_uint4(o32[0], o32[1], o32[2], o32[3]);
          if ((lane & 7) == 0) scaleBuf[e0 >> 7] = scale;
        }
      }
    }
    // shared-memory writes of every lane become visible to the bulk-copy engine
    ptx::fence_proxy_async_smem();
    __syncwarp();
    // ---- route: lane k owns the token's k-th expert.  It takes a row slot in the region this rank
    // owns on the expert's rank (local atomic: no cross-rank contention) and hands the row and the
    // scales to the copy engine of the SM as bulk copies straight into that rank's receive area.
    if (lane < a.topk) {
      const int k = lane;
      const int e = a.topkIdx[static_cast<size_t>(t) * a.topk + k];
      int slot = -1, dst = 0;
      if (e >= 0 && e < a.numExperts) {
        dst = e / a.expertsPerRank;
        slot = static_cast<int>(atomicAdd(a.sendCount + dst, 1u));
        if (slot >= a.rowsPerSource) {
          atomicAdd(a.overflow, 1u);
          slot = -1;
        }
      }
      a.slotOf[static_cast<size_t>(t) * a.topk + k] = slot < 0 ? -1 : ((dst << 24) | slot);
      if (slot >= 0) {
        const size_t r = static_cast<size_t>(me) * a.rowsPerSource + slot;
        ptx::bulk_store(a.recvX[dst] + r * H, rowBuf, static_cast<uint32_t>(H));
        float* sdst = a.recvScale[dst] + r * nblk;
        if (scalesBulk) {
          ptx::bulk_store(sdst, scaleBuf, scaleBytes);
        } else {
          for (int b = 0; b < nblk; ++b) sdst[b] = scaleBuf[b];
        }
        *reinterpret_cast<int4*>(a.recvMeta[dst] + r * 4) = make_int4(t, e - dst * a.expertsPerRank, k, 1);
      }
      ptx::tma_store_commit();
    }
  }
  // every bulk copy of this thread has completed (written, not just read) before the CTA reports in
  if (lane < a.topk) ptx::tma_store_wait<0>();

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

// TK = upper bound of top-k the instantiation handles; U iterations of 256 elements are in
// flight together (TK * U = 16 loads of 16 bytes per lane).
template <int TK, int U>
__global__ void __launch_bounds__(kMoeThreads) moe_combine_kernel(const __grid_constant__ MoeArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warpsPerCta = kMoeThreads / 32;
  const int me = a.dc.rank, H = a.hidden;
  const int iters = (H + 255) / 256;
  for (int t = blockIdx.x * warpsPerCta + warp; t < a.tokens; t += gridDim.x * warpsPerCta) {
    const char* src[TK];
    float w[TK];
#pragma unroll
    for (int k = 0; k < TK; ++k) {
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
    for (int i0 = 0; i0 < iters; i0 += U) {
      uint4 v[U][TK];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int el = (i0 + u) * 256 + lane * 8;
#pragma unroll
        for (int k = 0; k < TK; ++k)
          if (el < H && src[k]) v[u][k] = ptx::ld_stream_v4(src[k] + static_cast<size_t>(el) * 2);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int el = (i0 + u) * 256 + lane * 8;
        if (el >= H) continue;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < TK; ++k) {
          if (src[k]) {
            const uint32_t x[4] = {v[u][k].x, v[u][k].y, v[u][k].z, v[u][k].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 p = ptx::unpack_bf16x2(x[j]);
              acc[2 * j] += w[k] * p.x;
              acc[2 * j + 1] += w[k] * p.y;
            }
          }
        }
        ptx::st_global_v4(orow + static_cast<size_t>(el) * 2, Vec<DT_BF16>::pack(acc));
      }
    }
  }
}

}  // namespace dev

cudaError_t launchMoeDispatch(const MoeArgs& a, cudaStream_t stream) {
  if (a.hidden % 128 != 0 || a.hidden > 8192 || a.topk < 1 || a.topk > dev::kMoeMaxTopk) return cudaErrorInvalidValue;
  const int smem = (dev::kMoeThreads / 32) * dev::moe_warp_smem(a.hidden);
  static thread_local int attrDev = -1;
  int devId = 0;
  cudaGetDevice(&devId);
  if (attrDev != devId) {
    cudaError_t e = cudaFuncSetAttribute(dev::moe_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * dev::moe_warp_smem(8192));
    if (e != cudaSuccess) return e;
    attrDev = devId;
  }
  // as many CTAs as fit at once (shared memory allows three of the largest rows per SM); a warp
  // takes one token after the other
  int ctas = (a.tokens + 7) / 8;
  ctas = ctas < 1 ? 1 : (ctas > 444 ? 444 : ctas);
  dev::moe_dispatch_kernel<<<ctas, dev::kMoeThreads, smem, stream>>>(a);
  return cudaGetLastError();
}
cudaError_t launchMoeCombine(const MoeArgs& a, cudaStream_t stream) {
  if (a.hidden % 128 != 0 || a.hidden > dev::kMoeMaxIter * 256 || a.topk < 1 || a.topk > dev::kMoeMaxTopk)
    return cudaErrorInvalidValue;
  int ctas = (a.tokens + 7) / 8;
  ctas = ctas < 1 ? 1 : (ctas > 592 ? 592 : ctas);
  if (a.topk <= 4) dev::moe_combine_kernel<4, 4><<<ctas, dev::kMoeThreads, 0, stream>>>(a);
  else if (a.topk <= 8) dev::moe_combine_kernel<8, 2><<<ctas, dev::kMoeThreads, 0, stream>>>(a);
  else dev::moe_combine_kernel<16, 1><<<ctas, dev::kMoeThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace uccl
