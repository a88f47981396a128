// Expert-parallel all-to-all for mixture-of-experts layers: fp8 block-scaled dispatch and
// weighted bf16 combine over NVLink peer memory (see moe.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_comm.h"

namespace uccl {

struct MoeArgs {
  DevComm dc;
  int tokens;           // tokens of this rank in this call
  int hidden;           // multiple of 128, at most 8192
  int topk;             // at most 16
  int expertsPerRank;
  int numExperts;       // routing entries outside [0, numExperts) are unused slots
  int rowsPerSource;    // capacity of the region each source rank owns on every destination
  // symmetric receive area, one base pointer per rank
  char* recvX[UCCL_MAX_LOCAL_RANKS];       // fp8 [nranks][rowsPerSource][hidden]
  float* recvScale[UCCL_MAX_LOCAL_RANKS];  // [nranks][rowsPerSource][hidden / 128]
  int32_t* recvMeta[UCCL_MAX_LOCAL_RANKS]; // [nranks][rowsPerSource][4]
  int32_t* recvCounts[UCCL_MAX_LOCAL_RANKS];  // [nranks]
  uint32_t* arrived[UCCL_MAX_LOCAL_RANKS]; // [nranks] flag: source finished (epoch valued)
  const char* expertOut[UCCL_MAX_LOCAL_RANKS];  // bf16 [nranks][rowsPerSource][hidden]
  // local state
  uint32_t* sendCount;  // [nranks] rows handed to each destination in this call
  uint32_t* ctasDone;   // completion counter of the dispatch grid
  uint32_t* epoch;      // dispatch calls completed so far
  int32_t* slotOf;      // [maxTokens][topk]: (destination << 24) | row slot, or -1
  uint32_t* overflow;   // rows that did not fit rowsPerSource (should stay 0)
  // call arguments
  const void* x;        // bf16 [tokens, hidden]
  const int32_t* topkIdx;
  const float* topkWeight;
  void* out;            // bf16 [tokens, hidden]
};

cudaError_t launchMoeDispatch(const MoeArgs& a, cudaStream_t stream);
cudaError_t launchMoeCombine(const MoeArgs& a, cudaStream_t stream);

}  // namespace uccl
