// Kernel argument blocks and launch entry points of the NVLink-domain collectives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "device_comm.h"
#include "uccl.h"

namespace uccl {

// One launch of a collective over the NVLink domain.  `in[p]` / `out[p]` are rank p's
// peer-visible work buffers (the user's symmetric buffer, or the arena's staging area);
// `inUser` / `outUser` are set when data must first be copied into / finally out of the local
// work buffer because the user's buffer is not symmetric.
struct CollArgs {
  DevComm dc;
  const char* inUser;
  char* outUser;
  const char* in[UCCL_MAX_LOCAL_RANKS];
  char* out[UCCL_MAX_LOCAL_RANKS];
  const char* inMc;   // multicast alias of `in` (NVLS) or nullptr
  char* outMc;        // multicast alias of `out` or nullptr
  size_t bytes;       // all-reduce / broadcast / reduce: work bytes of this launch, 16-byte padded
  size_t userBytes;   // exact byte count behind `bytes` (or behind one chunk) in the user buffers
  size_t chunkBytes;  // chunked collectives: bytes per rank chunk in the work buffers
  size_t inStride;    // distance between consecutive rank chunks in inUser
  size_t outStride;   // distance between consecutive rank chunks in outUser
  int dtype;          // dev::DT_*
  int root;
  int vec;            // 1: every pointer/size is a 16-byte multiple
};

enum CollKernel : int {
  KERN_AR_ONESHOT = 0,
  KERN_AR_TWOSHOT = 1,
  KERN_AR_NVLS = 2,
  KERN_AR_LL = 3,
  KERN_AG_PULL = 4,
  KERN_AG_PUSH = 5,   // push with plain stores, or multimem.st when outMc is set
  KERN_RS_PULL = 6,   // pull with plain loads, or multimem.ld_reduce when inMc is set
  KERN_BCAST_PULL = 7,
  KERN_BCAST_PUSH = 8,
  KERN_REDUCE_PULL = 9,
  KERN_A2A_PULL = 10,
  KERN_BARRIER = 11,       // a rank barrier and nothing else (copy-engine mode)
  KERN_LOCAL_REDUCE = 12,  // out[0] = sum of `root` local slots of in[0], inStride apart
  KERN_RS_LL = 13,         // low-latency packets: inUser = [nranks][bytes] (inStride apart), outUser = my reduced chunk
  KERN_AG_LL = 14,         // low-latency packets: inUser = my chunk, outUser = [nranks][bytes] (outStride apart)
  KERN_A2A_LL = 15,        // low-latency packets: inUser and outUser = [nranks][bytes]
};

cudaError_t launchCollKernel(CollKernel k, const CollArgs& a, int blocks, cudaStream_t stream);

// Reduce-scatter with a scale and an output element type of its own, see fused_cast.cu.
struct CastArgs {
  DevComm dc;
  const char* in[UCCL_MAX_LOCAL_RANKS];  // every rank's input: nranks chunks, chunkStride bytes apart, peer-visible
  const char* inMc;                      // multicast alias of `in` (switch reduction) or nullptr
  const char* inUser;                    // set when `in` is the staging area: my input is copied in first
  size_t inStride;                       // bytes between consecutive rank chunks in inUser
  size_t chunkStride;                    // bytes between consecutive rank chunks in `in`
  size_t chunkElems;                     // elements per rank chunk in this launch
  int inType, outType;                   // ucclDataType_t
  float scale;
  char* out;                             // local: this rank's chunk in outType, 16-byte aligned
  float* outScales;                      // fp8 output: one scale per 128 elements
};
cudaError_t launchReduceCastKernel(const CastArgs& a, int blocks, cudaStream_t stream);

// Ring all-reduce / all-gather / reduce-scatter over peer-memory step FIFOs (Simple protocol)
// and the LL128 line protocol; see ring.cu.
struct RingArgs {
  DevComm dc;
  const char* inUser;
  char* outUser;
  size_t count;       // elements (all-reduce) or elements per rank chunk
  int dtype;
  int coll;           // ucclCollKind_t: AllReduce / AllGather / ReduceScatter
  int proto;          // ucclProtoSimple / ucclProtoLL128
  int ringPrev, ringNext;  // NVLink-domain indices of the ring neighbours
  int ringPos;        // my position in the ring order
  int ringRanks[UCCL_MAX_LOCAL_RANKS];  // ring order (position -> domain index)
  size_t ringBufOff;  // Simple protocol: offset of the step buffers inside the arena
  size_t ringBufBytes;  // and their total size (split evenly over the channels)
};
cudaError_t launchRingKernel(const RingArgs& a, int blocks, cudaStream_t stream);

// Point-to-point: each entry is one send or one receive through the receiver's arena slots.
// Operations with the same peer and the same direction share one FIFO, so they form a chain that
// one set of CTAs runs in order (`next`); different chains run side by side.
struct P2pOp {
  int isSend;
  int peer;       // NVLink-domain index
  int next;       // next operation of the same (peer, direction) chain in this launch, or -1
  int pad;
  const char* src;
  char* dst;
  size_t bytes;
};
constexpr int kMaxP2pChains = 2 * UCCL_MAX_LOCAL_RANKS;  // (peer, direction) pairs
constexpr int kP2pChainDepth = 2;                        // operations of one chain per launch
constexpr int kMaxP2pOps = kMaxP2pChains * kP2pChainDepth;
struct P2pArgs {
  DevComm dc;
  int nchains;
  int heads[kMaxP2pChains];  // first operation of every chain
  P2pOp ops[kMaxP2pOps];
};
cudaError_t launchP2pKernel(const P2pArgs& a, cudaStream_t stream);

// Fused all-reduce + residual add + RMSNorm, see fused_norm.cu.
struct ArNormArgs {
  DevComm dc;
  const char* in[UCCL_MAX_LOCAL_RANKS];  // every rank's partial sums [tokens, hidden] bf16, peer-visible
  const char* inMc;                      // multicast alias of `in` or nullptr
  const char* inUser;                    // set when `in` is the staging area: copy from here first
  const __nv_bfloat16* residual;         // [tokens, hidden], local
  const __nv_bfloat16* gamma;            // [hidden]
  char* outLocal;                        // normalised output [tokens, hidden], local
  char* resOut[UCCL_MAX_LOCAL_RANKS];    // every rank's new residual stream, peer-visible
  char* resOutMc;
  char* resOutUser;                      // set when `resOut` is the staging area: copy there last
  int tokens, hidden;
  float eps;
  int mcRows;  // switch path: rows per pass of the all-reduce phase (1, 2 or 4), own rows normalised in phase B; 0 = from registers, one row per pass
  int debug;  // experiment switches (UCCL_NORM_DEBUG): 1 no phase B, 2 no phase-A stores, 4 no phase A
};
cudaError_t launchArNormKernel(const ArNormArgs& a, int blocks, cudaStream_t stream);

}  // namespace uccl
