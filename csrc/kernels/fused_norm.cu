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

#ifdef UCCL_EXPERIMENTS
#define UCCL_NORM_DBG(a, bit) (((a).debug & (bit)) != 0)  // leave a phase out to time the rest (benchmarks/fused_layers.py)
#else
#define UCCL_NORM_DBG(a, bit) false
#endif

namespace uccl {
namespace dev {

constexpr int kNormMaxVec = 4;  // 16-byte vectors per thread and row: hidden <= 4 * 512 * 8 = 16384
constexpr int kNormSlots = 8;   // 16-byte vectors a thread keeps in flight: rows per pass x vectors per row
constexpr int kNormMaxRows = 4; // rows a CTA works on per pass

// Sums R per-row partials over the CTA in one pass (two barriers for all rows together).
__device__ __forceinline__ void block_sum_rows(float (&v)[kNormMaxRows]) {
  __shared__ float red[kNormMaxRows][kThreads / 32];
  __shared__ float total[kNormMaxRows];
#pragma unroll
  for (int j = 0; j < kNormMaxRows; ++j)
    for (int o = 16; o > 0; o >>= 1) v[j] += __shfl_xor_sync(0xffffffffu, v[j], o);
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int j = 0; j < kNormMaxRows; ++j) red[j][threadIdx.x >> 5] = v[j];
  }
  __syncthreads();
  if (threadIdx.x < 32 * kNormMaxRows) {
    const int j = threadIdx.x >> 5, l = threadIdx.x & 31;
    float t = l < kThreads / 32 ? red[j][l] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (l == 0) total[j] = t;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kNormMaxRows; ++j) v[j] = total[j];
  __syncthreads();
}

// One pass = R rows (R * nvecThread <= kNormSlots).  Slot s of a thread is vector s % nvecThread
// of row s / nvecThread of the pass.
struct NormPass {
  int nvecThread;  // vectors per thread and row
  int R;           // rows per pass
  __device__ __forceinline__ bool slot(int s, int rowsHere, int* j, int* v) const {
    *j = s / nvecThread;
    *v = threadIdx.x + (s - *j * nvecThread) * kThreads;
    return *j < rowsHere;
  }
};

// out rows = h * rsqrt(mean(h^2) + eps) * gamma for the rows of one pass held in registers
__device__ __forceinline__ void normalise_rows(const NormPass& np, const uint4 (&h)[kNormSlots], int rowsHere,
                                               const size_t (&rowIdx)[kNormMaxRows], const __nv_bfloat16* gamma, char* out,
                                               size_t rowBytes, float eps, int hidden) {
  const int vecPerRow = hidden >> 3;
  float ss[kNormMaxRows] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < kNormSlots; ++s) {
    int j, v;
    if (np.slot(s, rowsHere, &j, &v)) {
      const uint32_t w[4] = {h[s].x, h[s].y, h[s].z, h[s].w};
      float t = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = ptx::unpack_bf16x2(w[e]);
        t += f.x * f.x + f.y * f.y;
      }
#pragma unroll
      for (int jj = 0; jj < kNormMaxRows; ++jj)
        if (jj == j) ss[jj] += t;
    }
  }
  block_sum_rows(ss);
#pragma unroll
  for (int s = 0; s < kNormSlots; ++s) {
    int j, v;
    if (np.slot(s, rowsHere, &j, &v) && v < vecPerRow) {
      float sum = ss[0];
#pragma unroll
      for (int jj = 1; jj < kNormMaxRows; ++jj)
        if (jj == j) sum = ss[jj];
      size_t row = rowIdx[0];
#pragma unroll
      for (int jj = 1; jj < kNormMaxRows; ++jj)
        if (jj == j) row = rowIdx[jj];
      const float rstd = rsqrtf(sum / static_cast<float>(hidden) + eps);
      const uint4 g = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(gamma) + (static_cast<size_t>(v) << 4));
      const uint32_t w[4] = {h[s].x, h[s].y, h[s].z, h[s].w};
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = ptx::unpack_bf16x2(w[e]);
        const float2 gg = ptx::unpack_bf16x2(gw[e]);
        o[e] = ptx::pack_bf16x2(f.x * rstd * gg.x, f.y * rstd * gg.y);
      }
      ptx::st_global_v4(out + row * rowBytes + (static_cast<size_t>(v) << 4), make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

__device__ __forceinline__ uint4 add_bf16x8(uint4 x, uint4 y) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  Vec<DT_BF16>::add(acc, x);
  Vec<DT_BF16>::add(acc, y);
  return Vec<DT_BF16>::pack(acc);
}

__global__ void __launch_bounds__(kThreads, 1) ar_norm_kernel(const __grid_constant__ ArNormArgs a) {
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x, n = dc.nranks, me = dc.rank;
  const int vecPerRow = a.hidden >> 3;
  const size_t rowBytes = static_cast<size_t>(a.hidden) * 2;
  const int perRow = (vecPerRow + kThreads - 1) / kThreads;  // slots per row (same for every thread)
  NormPass np;
  np.nvecThread = perRow;
  np.R = min(kNormMaxRows, kNormSlots / perRow);

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
  // ---- phase A: my rows (rows b, b+B, ... of my shard).  Through the switch one row per pass is
  // enough to cover the latency (the links, not the loads in flight, are the limit) and lets the
  // stores of one pass travel while the loads of the next are already out; the peer path takes R.
  const NormPass npB = np;
  // Through the switch phase A is a plain all-reduce loop over this rank's rows (reduce in the
  // switch, add the residual, broadcast through the switch), as many rows in flight as the
  // registers hold and no CTA-wide reduction in between; the rows are normalised in phase B with
  // everybody else's, from local memory.  mcRows = 1, 2 or 4 rows per pass, 0 = the older form
  // that normalises its own rows from registers one row per pass.
  const bool splitNorm = a.inMc && a.resOutMc && a.mcRows > 0;
  if (a.inMc) np.R = splitNorm ? max(1, min(np.R, a.mcRows)) : 1;
  for (size_t r0 = b; r0 < (UCCL_NORM_DBG(a, 4) ? 0 : myLen); r0 += static_cast<size_t>(B) * np.R) {
    size_t rowIdx[kNormMaxRows];
    int rowsHere = 0;
#pragma unroll
    for (int j = 0; j < kNormMaxRows; ++j) {
      const size_t r = r0 + static_cast<size_t>(j) * B;
      rowIdx[j] = myOff + (r < myLen ? r : r0);
      if (j < np.R && r < myLen) rowsHere = j + 1;
    }
    uint4 h[kNormSlots], res[kNormSlots];
    // all loads of the pass are issued before the first use
#pragma unroll
    for (int s = 0; s < kNormSlots; ++s) {
      int j, v;
      if (np.slot(s, rowsHere, &j, &v) && v < vecPerRow) {
        size_t row = rowIdx[0];
#pragma unroll
        for (int jj = 1; jj < kNormMaxRows; ++jj)
          if (jj == j) row = rowIdx[jj];
        const size_t off = row * rowBytes + (static_cast<size_t>(v) << 4);
        if (a.inMc) {
          h[s] = ptx::multimem_ld_reduce_bf16x8(a.inMc + off);
        } else {
          float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int p = 0; p < n; ++p) Vec<DT_BF16>::add(acc, ptx::ld_stream_v4(a.in[(me + p) % n] + off));
          h[s] = Vec<DT_BF16>::pack(acc);
        }
        res[s] = ptx::ld_global_v4(reinterpret_cast<const char*>(a.residual) + off);
      } else {
        h[s] = make_uint4(0, 0, 0, 0);
        res[s] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int s = 0; s < kNormSlots; ++s) {
      int j, v;
      if (np.slot(s, rowsHere, &j, &v) && v < vecPerRow) {
        size_t row = rowIdx[0];
#pragma unroll
        for (int jj = 1; jj < kNormMaxRows; ++jj)
          if (jj == j) row = rowIdx[jj];
        const size_t off = row * rowBytes + (static_cast<size_t>(v) << 4);
        h[s] = add_bf16x8(h[s], res[s]);
        if (UCCL_NORM_DBG(a, 2)) {
        } else if (a.resOutMc) {
          ptx::multimem_st_v4(a.resOutMc + off, h[s]);
        } else {
          for (int p = 0; p < n; ++p) ptx::st_global_v4(a.resOut[(me + p) % n] + off, h[s]);
        }
      }
    }
    if (!splitNorm) normalise_rows(np, h, rowsHere, rowIdx, a.gamma, a.outLocal, rowBytes, a.eps, a.hidden);
  }
  if (!rank_barrier(dc)) return;
  // ---- phase B: rows owned by the other ranks, now present in my copy of the residual stream
  for (int q = splitNorm ? 0 : 1; q < (UCCL_NORM_DBG(a, 1) ? 0 : n); ++q) {
    const int p = (me + q) % n;
    size_t ro, rl;
    split(static_cast<size_t>(a.tokens), n, p, &ro, &rl);
    for (size_t r0 = b; r0 < rl; r0 += static_cast<size_t>(B) * npB.R) {
      size_t rowIdx[kNormMaxRows];
      int rowsHere = 0;
#pragma unroll
      for (int j = 0; j < kNormMaxRows; ++j) {
        const size_t r = r0 + static_cast<size_t>(j) * B;
        rowIdx[j] = ro + (r < rl ? r : r0);
        if (j < npB.R && r < rl) rowsHere = j + 1;
      }
      uint4 h[kNormSlots];
#pragma unroll
      for (int s = 0; s < kNormSlots; ++s) {
        int j, v;
        if (npB.slot(s, rowsHere, &j, &v) && v < vecPerRow) {
          size_t row = rowIdx[0];
#pragma unroll
          for (int jj = 1; jj < kNormMaxRows; ++jj)
            if (jj == j) row = rowIdx[jj];
          h[s] = ptx::ld_global_v4(a.resOut[me] + row * rowBytes + (static_cast<size_t>(v) << 4));
        } else {
          h[s] = make_uint4(0, 0, 0, 0);
        }
      }
      normalise_rows(npB, h, rowsHere, rowIdx, a.gamma, a.outLocal, rowBytes, a.eps, a.hidden);
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
  const int perRow = (vecPerRow + kThreads - 1) / kThreads;
  NormPass np;
  np.nvecThread = perRow;
  np.R = min(kNormMaxRows, kNormSlots / perRow);
  const size_t tokens = static_cast<size_t>(a.tokens);
  const int B = gridDim.x;
  for (size_t r0 = blockIdx.x; r0 < tokens; r0 += static_cast<size_t>(B) * np.R) {
    size_t rowIdx[kNormMaxRows];
    int rowsHere = 0;
#pragma unroll
    for (int j = 0; j < kNormMaxRows; ++j) {
      const size_t r = r0 + static_cast<size_t>(j) * B;
      rowIdx[j] = r < tokens ? r : r0;
      if (j < np.R && r < tokens) rowsHere = j + 1;
    }
    uint4 h[kNormSlots], res[kNormSlots];
#pragma unroll
    for (int s = 0; s < kNormSlots; ++s) {
      int j, v;
      if (np.slot(s, rowsHere, &j, &v) && v < vecPerRow) {
        size_t row = rowIdx[0];
#pragma unroll
        for (int jj = 1; jj < kNormMaxRows; ++jj)
          if (jj == j) row = rowIdx[jj];
        const size_t off = row * rowBytes + (static_cast<size_t>(v) << 4);
        h[s] = ptx::ld_global_v4(a.inUser + off);
        res[s] = ptx::ld_global_v4(reinterpret_cast<const char*>(a.residual) + off);
      } else {
        h[s] = make_uint4(0, 0, 0, 0);
        res[s] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int s = 0; s < kNormSlots; ++s) {
      int j, v;
      if (np.slot(s, rowsHere, &j, &v) && v < vecPerRow) {
        size_t row = rowIdx[0];
#pragma unroll
        for (int jj = 1; jj < kNormMaxRows; ++jj)
          if (jj == j) row = rowIdx[jj];
        h[s] = add_bf16x8(h[s], res[s]);
        ptx::st_global_v4(a.resOutUser + row * rowBytes + (static_cast<size_t>(v) << 4), h[s]);
      }
    }
    normalise_rows(np, h, rowsHere, rowIdx, a.gamma, a.outLocal, rowBytes, a.eps, a.hidden);
  }
}

}  // namespace dev

cudaError_t launchArNormKernel(const ArNormArgs& a, int blocks, cudaStream_t stream) {
  // the multi-rank kernel has one cross-rank barrier slot per CTA
  if (a.hidden % 8 != 0 || a.hidden > dev::kNormMaxVec * dev::kThreads * 8 || blocks < 1 ||
      blocks > (a.dc.nranks <= 1 ? 1024 : kMaxBlocks))
    return cudaErrorInvalidValue;
  if (a.dc.nranks <= 1) dev::add_norm_kernel<<<blocks, dev::kThreads, 0, stream>>>(a);
  else dev::ar_norm_kernel<<<blocks, dev::kThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace uccl
