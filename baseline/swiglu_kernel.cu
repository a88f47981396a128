// One-pass SwiGLU for the NCCL + cuBLAS comparator: h[r, c] = silu(gu[r, c]) * gu[r, F + c] for a
// [rows, 2F] bf16 input, reading every element once and writing h once.  It belongs to the
// baseline, not to the library: the comparator's elementwise step should not be charged for three
// eager kernels with fresh allocations when one pass is what any serving stack would run.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__global__ void __launch_bounds__(256) swiglu_kernel(const uint4* __restrict__ gu, uint4* __restrict__ h, long rows, int vecPerHalf) {
  // one thread per 16-byte vector of the output (8 bf16)
  const long total = rows * vecPerHalf;
  for (long i = blockIdx.x * 256L + threadIdx.x; i < total; i += gridDim.x * 256L) {
    const long r = i / vecPerHalf;
    const int c = static_cast<int>(i - r * vecPerHalf);
    const uint4 g = gu[r * 2 * vecPerHalf + c];
    const uint4 u = gu[r * 2 * vecPerHalf + vecPerHalf + c];
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gf = __bfloat1622float2(gp[j]), uf = __bfloat1622float2(up[j]);
      op[j] = __floats2bfloat162_rn(gf.x / (1.f + __expf(-gf.x)) * uf.x, gf.y / (1.f + __expf(-gf.y)) * uf.y);
    }
    h[i] = o;
  }
}

}  // namespace

// F must be a multiple of 8; both pointers 16-byte aligned.  Returns a cudaError_t.
extern "C" int baselineSwiglu(const void* gu, void* h, long rows, int F, void* stream) {
  if (F % 8 != 0 || rows <= 0) return cudaErrorInvalidValue;
  const int vecPerHalf = F / 8;
  const long total = rows * vecPerHalf;
  const int blocks = static_cast<int>(total / 256 + 1 < 148L * 16 ? total / 256 + 1 : 148L * 16);
  swiglu_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(gu), static_cast<uint4*>(h), rows, vecPerHalf);
  return static_cast<int>(cudaGetLastError());
}
