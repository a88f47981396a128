// Host-side launcher interface of the tcgen05 GEMM (see gemm_sm100.cuh for the kernel).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "uccl.h"

namespace uccl {

struct GemmCommPlan;  // defined in gemm_sm100.cu next to the kernel argument structs

struct GemmLaunch {
  const void* A = nullptr;  // [M, K] bf16, row stride lda
  const void* B = nullptr;  // [N, K] bf16, row stride ldb
  void* C = nullptr;        // [M, N] (or [M, N/2] for SwiGLU) bf16, row stride ldc
  int M = 0, N = 0, K = 0;
  int lda = 0, ldb = 0, ldc = 0;
  int epilogue = 0;         // 0 store, 1 SwiGLU
  int max_ctas = 0;         // 0 = one per SM
  uint32_t* err = nullptr;  // optional device-visible error word
};

// Fusion descriptor filled by the tensor-parallel entry points.
struct GemmFusion {
  int role = 0;  // 0 none, 1 all-gather, 2 reduce-scatter (TMA push + local sum), 3 reduce-scatter (copy engines + local sum)
  int rank = 0, nranks = 1;
  int comm_ctas = 0;         // all-gather: CTAs that move data (reduce-scatter reserves none)
  uint64_t timeout_ns = 0;
  uint32_t* abort_flag = nullptr;
  // rank barrier folded into the launch (all three null: the caller ran a barrier kernel itself):
  // every rank's arena, this rank's epoch counters, and a local word that is zero at launch
  char* const* arena_peer = nullptr;
  uint32_t* epochs = nullptr;
  uint32_t* go = nullptr;
  int rows_per_rank = 0;
  // all-gather: my shard, every rank's A_full (peer-mapped) and every rank's arrival counters
  // (zeroed before the launch); a_inplace: the shard already sits in my A_full
  const void* a_shard = nullptr;
  int a_inplace = 0;
  int a_external = 0;  // the rows arrive by copy engines: no communication CTAs, flags are set to 1
  int a_peer_major = 0;  // visit the other ranks' shards one rank after the other, nearest first (copy-engine lanes)
  int a_spread = 0;    // no communication CTAs either: a forwarder warp in every GEMM CTA pushes the shard
  void* a_full_peer[UCCL_MAX_LOCAL_RANKS] = {};
  uint32_t* ready_peer[UCCL_MAX_LOCAL_RANKS] = {};
  // reduce-scatter: every rank's staging buffer [nranks][rows_per_rank][N] (peer-mapped) and
  // per-row-block counters (zeroed before the launch); output of this rank
  void* stage_peer[UCCL_MAX_LOCAL_RANKS] = {};
  uint32_t* done_peer[UCCL_MAX_LOCAL_RANKS] = {};
  void* rs_out = nullptr;
  int rs_ldo = 0;
  // reduce-scatter: CTAs that do nothing but sum the staged copies while the others compute
  // (0 = every CTA computes first and sums afterwards); tail_next: local word, zero at launch
  int rs_reducers = 0;
  uint32_t* tail_next = nullptr;
};

ucclResult_t launchGemmBf16(const GemmLaunch& g, const GemmFusion* fusion, cudaStream_t stream);


// Number of SMs of the current device (cached per device).
int deviceSmCount();

}  // namespace uccl
