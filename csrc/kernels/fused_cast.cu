// Reduce-scatter with a fused epilogue: out[i] = cast(scale * sum over ranks of in_r[my chunk][i]).
//
// The sum is carried in fp32 registers from the peer loads to the store, so "sum, scale, change
// the element type" costs no extra pass over memory: bf16 / fp16 / fp32 in, bf16 / fp16 / fp32 or
// fp8-e4m3 out.  With fp8 output every 128 consecutive elements share one fp32 scale
// (amax / 448, the block layout the MoE dispatch uses), written next to the data.
// The reference adds in the 16-bit element type and has no cast or scale
// (src/device/reduce_kernel.hpp:17-20); its design notes list more element types as future work
// (desgin/design-spec.md:1759).
//
// Shape of the kernel (same as the other NVLink collectives): [copy my input into the staging
// area] -> rank barrier -> every CTA pulls its slice of this rank's chunk from all ranks (plain
// peer loads, eight in flight per thread, or multimem.ld_reduce through the switch), scales,
// converts and stores locally -> rank barrier (peers are done reading my memory).
// Work is cut in units of 128 elements so that an fp8 scale block never straddles two CTAs, and
// the 128 elements of a block sit in consecutive lanes of one warp (16 lanes for 16-bit input,
// 32 for fp32 input), which makes the block's amax a shuffle reduction.
#include <cuda_fp8.h>

#include "coll_device.cuh"
#include "collectives.cuh"

namespace uccl {
namespace dev {

enum : int { OUT_F16 = 0, OUT_BF16 = 1, OUT_F32 = 2, OUT_FP8 = 3 };

template <int OUT, int NE>
__device__ __forceinline__ void store_cast(char* out, size_t elem, const float (&v)[8]) {
  if (OUT == OUT_F32) {
    char* p = out + elem * 4;
    ptx::st_global_v4(p, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])));
    if (NE == 8)
      ptx::st_global_v4(p + 16, make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7])));
  } else if (OUT == OUT_BF16 || OUT == OUT_F16) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < NE / 2; ++j)
      w[j] = OUT == OUT_BF16 ? ptx::pack_bf16x2(v[2 * j], v[2 * j + 1]) : ptx::pack_f16x2(v[2 * j], v[2 * j + 1]);
    char* p = out + elem * 2;
    if (NE == 8) ptx::st_global_v4(p, make_uint4(w[0], w[1], w[2], w[3]));
    else *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
  }
}

// quantise with the block's scale (a true division, as in the MoE dispatch, so that the result is
// bit-identical to an fp32 restatement of the cast)
template <int NE>
__device__ __forceinline__ void store_fp8(char* out, size_t elem, const float (&v)[8], float blockScale) {
  uint32_t w[2] = {0, 0};
#pragma unroll
  for (int j = 0; j < NE / 4; ++j) {
    const __nv_fp8x2_storage_t a0 = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(v[4 * j], blockScale), __fdiv_rn(v[4 * j + 1], blockScale)), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t a1 = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(v[4 * j + 2], blockScale), __fdiv_rn(v[4 * j + 3], blockScale)), __NV_SATFINITE, __NV_E4M3);
    w[j] = static_cast<uint32_t>(a0) | (static_cast<uint32_t>(a1) << 16);
  }
  char* p = out + elem;
  if (NE == 8) *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
  else *reinterpret_cast<uint32_t*>(p) = w[0];
}

template <int DT, int OUT, bool NVLS>
__global__ void __launch_bounds__(kThreads, 1) reduce_cast_kernel(const __grid_constant__ CastArgs a) {
  using V = Vec<DT>;
  constexpr int NE = V::N;                 // elements per 16-byte input vector: 8 or 4
  constexpr int LANES = 128 / NE;          // lanes that share one 128-element block
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x, n = dc.nranks;
  const size_t vecPerChunk = (a.chunkElems + NE - 1) / NE;
  const size_t units = (a.chunkElems + 127) / 128;
  size_t u0, ul;
  split(units, B, b, &u0, &ul);
  const size_t v0 = u0 * LANES, v1 = min(vecPerChunk, (u0 + ul) * LANES);
  if (a.inUser) {
    // my contribution to every rank's chunk goes into the staging area, same slice as I will read
    for (int s = 0; s < n; ++s) {
      const size_t begin = v0 << 4, len = v1 > v0 ? (v1 - v0) << 4 : 0;
      const size_t userBytes = a.chunkElems * V::ES;
      if (begin < userBytes)
        block_copy(const_cast<char*>(a.in[dc.rank]) + s * a.chunkStride + begin, a.inUser + s * a.inStride + begin,
                   min(len, userBytes - begin));
    }
  }
  if (n > 1 && !rank_barrier(dc)) return;  // a single rank has no arena to meet in
  const size_t mine = static_cast<size_t>(dc.rank) * a.chunkStride;
  // whole warps run every iteration: lanes beyond the slice's last vector still take part in the shuffles
  const size_t vEnd = v1 > v0 ? v0 + ((v1 - v0 + 31) / 32) * 32 : v0;
  for (size_t v = v0 + threadIdx.x; v < vEnd; v += blockDim.x) {
    const bool live = v < v1;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (live) {
      const size_t off = mine + (v << 4);
      if (NVLS) {
        V::add(acc, V::mc_reduce(a.inMc + off));
      } else {
        uint4 d[8];
        for (int p0 = 0; p0 < n; p0 += 8) {
          const int m = min(8, n - p0);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < m) d[j] = ptx::ld_stream_v4(a.in[(dc.rank + p0 + j) % n] + off);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < m) V::add(acc, d[j]);
        }
      }
#pragma unroll
      for (int e = 0; e < NE; ++e) acc[e] *= a.scale;
    }
    const size_t elem = v * NE;
    if (OUT == OUT_FP8) {
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < NE; ++e) amax = fmaxf(amax, fabsf(acc[e]));
#pragma unroll
      for (int o = LANES / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float blockScale = fmaxf(amax, 1e-10f) / 448.f;
      if (live) {
        store_fp8<NE>(a.out, elem, acc, blockScale);
        if ((v % LANES) == 0) a.outScales[v / LANES] = blockScale;
      }
    } else if (live) {
      store_cast<OUT, NE>(a.out, elem, acc);
    }
  }
  if (n > 1) rank_barrier(dc);
}

}  // namespace dev

template <int DT, bool NVLS>
static cudaError_t launchOut(const CastArgs& a, int blocks, cudaStream_t s) {
  switch (a.outType) {
    case ucclFloat16: dev::reduce_cast_kernel<DT, dev::OUT_F16, NVLS><<<blocks, dev::kThreads, 0, s>>>(a); break;
    case ucclBfloat16: dev::reduce_cast_kernel<DT, dev::OUT_BF16, NVLS><<<blocks, dev::kThreads, 0, s>>>(a); break;
    case ucclFloat32: dev::reduce_cast_kernel<DT, dev::OUT_F32, NVLS><<<blocks, dev::kThreads, 0, s>>>(a); break;
    case ucclFloat8e4m3: dev::reduce_cast_kernel<DT, dev::OUT_FP8, NVLS><<<blocks, dev::kThreads, 0, s>>>(a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launchReduceCastKernel(const CastArgs& a, int blocks, cudaStream_t s) {
  if (blocks < 1 || blocks > kMaxBlocks) return cudaErrorInvalidValue;
  const bool nvls = a.inMc != nullptr;
  switch (a.inType) {
    case ucclFloat16: return nvls ? launchOut<dev::DT_F16, true>(a, blocks, s) : launchOut<dev::DT_F16, false>(a, blocks, s);
    case ucclBfloat16: return nvls ? launchOut<dev::DT_BF16, true>(a, blocks, s) : launchOut<dev::DT_BF16, false>(a, blocks, s);
    case ucclFloat32: return nvls ? launchOut<dev::DT_F32, true>(a, blocks, s) : launchOut<dev::DT_F32, false>(a, blocks, s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace uccl
