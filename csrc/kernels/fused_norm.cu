// Fused all-reduce + residual add + RMSNorm for tensor-parallel layers (bf16).
//
//   h   = sum over ranks of x_r + residual          (kept as the new residual stream)
//   out = h * rsqrt(mean(h^2) + eps) * gamma
//
// The reference has no fused epilogues.  The library baseline is an all-reduce followed by a
// separate normalisation kernel: the reduced tensor crosses NVLink twice (reduce-scatter and
// all-gather halves) and is then read and written once more from HBM.  Here the token rows are
// sharded over the ranks:
//   phase A  each rank reduces its own rows (multimem.ld_reduce in the switch, or peer loads),
//            adds the residual, rounds to bf16 and stores the new residual row into every rank
//            (multimem.st, or peer stores); it normalises those rows while they are in registers;
//   phase B  after a rank barrier every rank normalises the rows it received, reading each once.
// Only one tensor travels the all-gather direction; the normalised output never crosses NVLink.
// CTA b handles rows b, b+B, ... of every shard in both phases, so the CTA-level rank barrier
// covers exactly the rows it later reads.
#include "coll_device.cuh"
#include "collectives.cuh"

namespace uccl {
namespace dev {

constexpr int kNormMaxVec = 4;  // 16-byte vectors per thread: hidden <= 4 * 512 * 8 = 16384

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float red[kThreads / 32];
  __shared__ float total;
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < kThreads / 32 ? red[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) total = t;
  }
  __syncthreads();
  const float r = total;
  __syncthreads();
  return r;
}

__device__ __forceinline__ void normalise_row(const uint4 (&h)[kNormMaxVec], int nvecThread, int vecPerRow,
                                              const __nv_bfloat16* gamma, char* outRow, float eps, int hidden) {
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kNormMaxVec; ++k) {
    if (k < nvecThread) {
      const uint32_t w[4] = {h[k].x, h[k].y, h[k].z, h[k].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = ptx::unpack_bf16x2(w[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(ss) / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int k = 0; k < kNormMaxVec; ++k) {
    if (k < nvecThread) {
      const int v = threadIdx.x + k * kThreads;
      const uint4 g = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(gamma) + (static_cast<size_t>(v) << 4));
      const uint32_t w[4] = {h[k].x, h[k].y, h[k].z, h[k].w};
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = ptx::unpack_bf16x2(w[j]);
        const float2 gg = ptx::unpack_bf16x2(gw[j]);
        o[j] = ptx::pack_bf16x2(f.x * rstd * gg.x, f.y * rstd * gg.y);
      }
      ptx::st_global_v4(outRow + (static_cast<size_t>(v) << 4), make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
  (void)vecPerRow;
}

__global__ void __launch_bounds__(kThreads, 1) ar_norm_kernel(const __grid_constant__ ArNormArgs a) {
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x, n = dc.nranks, me = dc.rank;
  const int vecPerRow = a.hidden >> 3;
  const size_t rowBytes = static_cast<size_t>(a.hidden) * 2;
  int nvecThread = 0;
  for (int v = threadIdx.x; v < vecPerRow; v += kThreads) ++nvecThread;

  // staged input: CTA b copies the rows it will be asked for by peers (rows b, b+B, ... of every shard)
  if (a.inUser) {
    for (int p = 0; p < n; ++p) {
      size_t ro, rl;
      split(static_cast<size_t>(a.tokens), n, p, &ro, &rl);
      for (size_t r = b; r < rl; r += B)
        block_copy(const_cast<char*>(a.in[me]) + (ro + r) * rowBytes, a.inUser + (ro + r) * rowBytes, rowBytes);
    }
  }
  if (!rank_barrier(dc)) return;

  size_t myOff, myLen;
  split(static_cast<size_t>(a.tokens), n, me, &myOff, &myLen);
  // ---- phase A: my rows
  for (size_t r = b; r < myLen; r += B) {
    const size_t row = myOff + r;
    uint4 h[kNormMaxVec];
#pragma unroll
    for (int k = 0; k < kNormMaxVec; ++k) {
      if (k < nvecThread) {
        const size_t off = row * rowBytes + (static_cast<size_t>(threadIdx.x + k * kThreads) << 4);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (a.inMc) {
          Vec<DT_BF16>::add(acc, ptx::multimem_ld_reduce_bf16x8(a.inMc + off));
        } else {
          for (int p = 0; p < n; ++p) Vec<DT_BF16>::add(acc, ptx::ld_stream_v4(a.in[(me + p) % n] + off));
        }
        Vec<DT_BF16>::add(acc, ptx::ld_global_v4(reinterpret_cast<const char*>(a.residual) + off));
        h[k] = Vec<DT_BF16>::pack(acc);
        if (a.resOutMc) {
          ptx::multimem_st_v4(a.resOutMc + off, h[k]);
        } else {
          for (int p = 0; p < n; ++p) ptx::st_global_v4(a.resOut[(me + p) % n] + off, h[k]);
        }
      }
    }
    normalise_row(h, nvecThread, vecPerRow, a.gamma, a.outLocal + row * rowBytes, a.eps, a.hidden);
  }
  if (!rank_barrier(dc)) return;
  // ---- phase B: rows owned by the other ranks, now present in my copy of the residual stream
  for (int q = 1; q < n; ++q) {
    const int p = (me + q) % n;
    size_t ro, rl;
    split(static_cast<size_t>(a.tokens), n, p, &ro, &rl);
    for (size_t r = b; r < rl; r += B) {
      const size_t row = ro + r;
      uint4 h[kNormMaxVec];
#pragma unroll
      for (int k = 0; k < kNormMaxVec; ++k)
        if (k < nvecThread)
          h[k] = ptx::ld_global_v4(a.resOut[me] + row * rowBytes + (static_cast<size_t>(threadIdx.x + k * kThreads) << 4));
      normalise_row(h, nvecThread, vecPerRow, a.gamma, a.outLocal + row * rowBytes, a.eps, a.hidden);
    }
  }
  // staged residual: hand the rows back to the user's buffer
  if (a.resOutUser) {
    for (int p = 0; p < n; ++p) {
      size_t ro, rl;
      split(static_cast<size_t>(a.tokens), n, p, &ro, &rl);
      for (size_t r = b; r < rl; r += B)
        block_copy(a.resOutUser + (ro + r) * rowBytes, a.resOut[me] + (ro + r) * rowBytes, rowBytes);
    }
  }
}

// single-rank / reference path: out = rmsnorm(x + residual) * gamma without any communication
__global__ void __launch_bounds__(kThreads, 1) add_norm_kernel(const __grid_constant__ ArNormArgs a) {
  const int vecPerRow = a.hidden >> 3;
  const size_t rowBytes = static_cast<size_t>(a.hidden) * 2;
  int nvecThread = 0;
  for (int v = threadIdx.x; v < vecPerRow; v += kThreads) ++nvecThread;
  for (size_t row = blockIdx.x; row < static_cast<size_t>(a.tokens); row += gridDim.x) {
    uint4 h[kNormMaxVec];
#pragma unroll
    for (int k = 0; k < kNormMaxVec; ++k) {
      if (k < nvecThread) {
        const size_t off = row * rowBytes + (static_cast<size_t>(threadIdx.x + k * kThreads) << 4);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        Vec<DT_BF16>::add(acc, ptx::ld_global_v4(a.inUser + off));
        Vec<DT_BF16>::add(acc, ptx::ld_global_v4(reinterpret_cast<const char*>(a.residual) + off));
        h[k] = Vec<DT_BF16>::pack(acc);
        ptx::st_global_v4(a.resOutUser + off, h[k]);
      }
    }
    normalise_row(h, nvecThread, vecPerRow, a.gamma, a.outLocal + row * rowBytes, a.eps, a.hidden);
  }
}

}  // namespace dev

cudaError_t launchArNormKernel(const ArNormArgs& a, int blocks, cudaStream_t stream) {
  if (a.hidden % 8 != 0 || a.hidden > dev::kNormMaxVec * dev::kThreads * 8 || blocks < 1 || blocks > kMaxBlocks)
    return cudaErrorInvalidValue;
  if (a.dc.nranks <= 1) dev::add_norm_kernel<<<blocks, dev::kThreads, 0, stream>>>(a);
  else dev::ar_norm_kernel<<<blocks, dev::kThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace uccl
