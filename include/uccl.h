/*
 * uccl.h -- public C interface of the Blackwell-native unified collective library.
 *
 * The entry points and enum values that the upstream unified-ccl project exposes
 * (src/include/uccl.h:15-146 and src/include/uccl_common.h:14-62 there) keep their names,
 * argument order and numeric values so that existing callers re-link without edits.  The
 * `stream` argument is a cudaStream_t passed as void* (NULL = the legacy default stream);
 * for a communicator created on the CPU backend it is ignored and calls are synchronous.
 *
 * Everything below the "extensions" banners is new: more collectives, point-to-point,
 * symmetric-memory allocation, fused compute+collective kernels, tuning and counters.
 */
#ifndef UCCL_PUBLIC_H_
#define UCCL_PUBLIC_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ version */
#define UCCL_MAJOR 0
#define UCCL_MINOR 1
#define UCCL_PATCH 0
#define UCCL_VERSION (UCCL_MAJOR * 10000 + UCCL_MINOR * 100 + UCCL_PATCH)

/* ------------------------------------------------------------------ limits */
#define UCCL_UNIQUE_ID_BYTES 128
#define UCCL_MAX_CHANNELS 16
#define UCCL_MAX_RANKS 128
#define UCCL_STEPS 8            /* in-flight slots per network FIFO                */
#define UCCL_MAX_LOCAL_RANKS 16 /* ranks that can share one NVLink symmetric heap  */

/* pointer kinds a network plugin can accept */
#define UCCL_PTR_HOST 0x1
#define UCCL_PTR_DEVICE 0x2

/* ------------------------------------------------------------------ enums */
typedef enum {
  ucclSuccess = 0,
  ucclSystemError = 1,
  ucclInternalError = 2,
  ucclInvalidArgument = 3,
  ucclInvalidUsage = 4,
  ucclRemoteError = 5,
  ucclInProgress = 6,
  ucclNumResults = 7
} ucclResult_t;

typedef enum {
  ucclFloat16 = 0,
  ucclBfloat16 = 1,
  /* extensions: appended so the two upstream values keep their meaning */
  ucclFloat32 = 2,
  ucclFloat8e4m3 = 3, /* copy-only collectives; reductions take block scales, see MoE */
  ucclUint8 = 4,      /* raw bytes, copy-only collectives                            */
  ucclNumTypes = 5
} ucclDataType_t;

typedef enum { ucclSum = 0, ucclNumOps = 1 } ucclRedOp_t;

/* algorithm / protocol identifiers (UCCL_ALGO / UCCL_PROTO accept the lower-case names) */
typedef enum {
  ucclAlgoAuto = 0,
  ucclAlgoRing = 1,
  ucclAlgoOneShot = 2,
  ucclAlgoTwoShot = 3,   /* "symmetric": pull-reduce my shard, push result to all */
  ucclAlgoNvls = 4,      /* multimem.ld_reduce / multimem.st through NVSwitch     */
  ucclAlgoCopyEngine = 5,
  ucclAlgoNet = 6,       /* proxy thread + network plugin                         */
  ucclNumAlgos = 7
} ucclAlgo_t;

typedef enum { ucclProtoAuto = 0, ucclProtoSimple = 1, ucclProtoLL = 2, ucclProtoLL128 = 3, ucclNumProtos = 4 } ucclProto_t;

/* ------------------------------------------------------------------ handles */
typedef struct ucclComm* ucclComm_t;
#define UCCL_COMM_NULL NULL
typedef struct { char internal[UCCL_UNIQUE_ID_BYTES]; } ucclUniqueId;
typedef struct ucclWindow* ucclWindow_t;

/* ------------------------------------------------------------------ lifecycle */
ucclResult_t ucclGetVersion(int* version);
/* Starts a rendezvous service in the calling process and encodes its address in the id. */
ucclResult_t ucclGetUniqueId(ucclUniqueId* uniqueId);
/* For launchers that already hand every rank a rendezvous address (MASTER_ADDR / MASTER_PORT):
 * all ranks derive the same id from (ip, port, seed); exactly one of them also calls
 * ucclServeUniqueId to run the rendezvous service there. */
ucclResult_t ucclUniqueIdFromAddress(const char* ip, int port, uint64_t seed, ucclUniqueId* uniqueId);
ucclResult_t ucclServeUniqueId(const ucclUniqueId* uniqueId);
ucclResult_t ucclCommInitRank(ucclComm_t* comm, int nranks, ucclUniqueId commId, int rank);
/* One process, ndev communicators (one per entry of devlist, or devices 0..ndev-1). */
ucclResult_t ucclCommInitAll(ucclComm_t* comm, int ndev, const int* devlist);
ucclResult_t ucclCommFinalize(ucclComm_t comm);
ucclResult_t ucclCommDestroy(ucclComm_t comm);
ucclResult_t ucclCommAbort(ucclComm_t comm);
ucclResult_t ucclCommCount(const ucclComm_t comm, int* count);
ucclResult_t ucclCommUserRank(const ucclComm_t comm, int* rank);

/* ------------------------------------------------------------------ collectives */
ucclResult_t ucclAllReduce(const void* sendbuff, void* recvbuff, size_t count,
                           ucclDataType_t datatype, ucclRedOp_t op, ucclComm_t comm, void* stream);
/* recvbuff holds sendcount * nranks elements */
ucclResult_t ucclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount,
                           ucclDataType_t datatype, ucclComm_t comm, void* stream);
/* sendbuff holds recvcount * nranks elements */
ucclResult_t ucclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount,
                               ucclDataType_t datatype, ucclRedOp_t op, ucclComm_t comm,
                               void* stream);

/* ------------------------------------------------------------------ collectives with a fused epilogue
 * out = cast<outType>(scale * sum over ranks(in)): the sum is carried in fp32 from the peer loads
 * to the store, so scaling and changing the element type cost no extra pass over memory.
 * inType: fp16 / bf16 / fp32.  outType: fp16 / bf16 / fp32, or fp8-e4m3, in which case every 128
 * consecutive elements share one fp32 scale (amax / 448) written to blockScales.
 * Buffers are 16-byte aligned; recvcount (count / nranks for the all-reduce) is a multiple of one
 * 16-byte input vector, of 128 for fp8 output.  Not deferrable into a group. */
ucclResult_t ucclReduceScatterEx(const void* sendbuff, void* recvbuff, size_t recvcount,
                                 ucclDataType_t inType, ucclDataType_t outType, float scale,
                                 float* blockScales, ucclComm_t comm, void* stream);
ucclResult_t ucclAllReduceEx(const void* sendbuff, void* recvbuff, size_t count, ucclDataType_t inType,
                             ucclDataType_t outType, float scale, float* blockScales, ucclComm_t comm,
                             void* stream);

/* ------------------------------------------------------------------ group */
ucclResult_t ucclGroupStart(void);
ucclResult_t ucclGroupEnd(void);

/* ------------------------------------------------------------------ RMA windows */
ucclResult_t ucclCommWindowRegister(ucclWindow_t* win, void* buff, size_t size, ucclComm_t comm);
ucclResult_t ucclCommWindowDeregister(ucclWindow_t win);

ucclResult_t ucclPut(const void* localBuff, size_t count, ucclDataType_t datatype, int peer,
                     ucclWindow_t peerWin, size_t peerWinOffset, ucclComm_t comm, void* stream);
ucclResult_t ucclGet(void* localBuff, size_t count, ucclDataType_t datatype, int peer,
                     ucclWindow_t peerWin, size_t peerWinOffset, ucclComm_t comm, void* stream);
ucclResult_t ucclPutSignal(const void* localBuff, size_t count, ucclDataType_t datatype, int peer,
                           ucclWindow_t peerWin, size_t peerWinOffset, int sigIdx, int ctx,
                           unsigned int flags, ucclComm_t comm, void* stream);
ucclResult_t ucclGetSignal(void* localBuff, size_t count, ucclDataType_t datatype, int peer,
                           ucclWindow_t peerWin, size_t peerWinOffset, int sigIdx, int ctx,
                           unsigned int flags, ucclComm_t comm, void* stream);
/* Raises signal counter (sigIdx) that `peer` keeps for this rank, in the window most recently
 * registered on the communicator. */
ucclResult_t ucclSignal(int peer, int sigIdx, int ctx, unsigned int flags, ucclComm_t comm,
                        void* stream);

typedef struct {
  int opCnt;        /* absolute number of signals expected from `peer` so far */
  int peer;
  int sigIdx;       /* must be 0 */
  int ctx;          /* must be 0 */
  ucclWindow_t win; /* window whose signal counters are waited on */
} ucclWaitSignalDesc_t;

ucclResult_t ucclWaitSignal(int nDesc, ucclWaitSignalDesc_t* signalDescs, ucclComm_t comm,
                            void* stream);

/* ------------------------------------------------------------------ errors */
const char* ucclGetErrorString(ucclResult_t result);
const char* ucclGetLastError(ucclComm_t comm);

/* ==================================================================
 * extensions: collectives and point-to-point
 * ================================================================== */
ucclResult_t ucclBroadcast(const void* sendbuff, void* recvbuff, size_t count,
                           ucclDataType_t datatype, int root, ucclComm_t comm, void* stream);
ucclResult_t ucclReduce(const void* sendbuff, void* recvbuff, size_t count,
                        ucclDataType_t datatype, ucclRedOp_t op, int root, ucclComm_t comm,
                        void* stream);
/* every rank sends `count` elements to every rank; both buffers hold count * nranks */
ucclResult_t ucclAllToAll(const void* sendbuff, void* recvbuff, size_t count,
                          ucclDataType_t datatype, ucclComm_t comm, void* stream);
ucclResult_t ucclSend(const void* sendbuff, size_t count, ucclDataType_t datatype, int peer,
                      ucclComm_t comm, void* stream);
ucclResult_t ucclRecv(void* recvbuff, size_t count, ucclDataType_t datatype, int peer,
                      ucclComm_t comm, void* stream);

/* Asynchronous error state: device-side wait expiry, proxy/network failure, abort. */
ucclResult_t ucclCommGetAsyncError(ucclComm_t comm, ucclResult_t* asyncError);

/* ==================================================================
 * extensions: symmetric memory
 * ================================================================== */
/* Collective: every rank of the node calls with the same size.  The returned device pointer
 * is backed by CUDA VMM memory that every local peer has mapped, and by an NVSwitch multicast
 * object when the hardware offers one.  Collectives on such buffers run zero-copy. */
ucclResult_t ucclMemAlloc(void** ptr, size_t size, ucclComm_t comm);
ucclResult_t ucclMemFree(void* ptr, ucclComm_t comm);
/* Collective.  With UCCL_CANARY=1 every buffer of ucclMemAlloc sits between painted guard regions;
 * this call synchronises the device and the ranks and verifies them all (ucclInternalError and a
 * message with the buffer and the byte offset when one was overwritten).  ucclMemFree checks the
 * buffer it releases the same way.  Without UCCL_CANARY it returns ucclSuccess. */
ucclResult_t ucclMemCheck(ucclComm_t comm);
/* Peer-mapped alias of a symmetric pointer (NULL result if `ptr` is not symmetric). */
ucclResult_t ucclMemPeerPointer(const void* ptr, int peer, ucclComm_t comm, void** peerPtr);
/* Multicast alias of a symmetric pointer (NULL result without NVLS). */
ucclResult_t ucclMemMulticastPointer(const void* ptr, ucclComm_t comm, void** mcPtr);

/* ==================================================================
 * extensions: fused compute + collective kernels (bf16)
 * ================================================================== */
/* out = RMSNorm(allreduce(x) + residual) * gamma ; residual_out = allreduce(x) + residual.
 * x: [tokens, hidden] partial sums of this rank.  residual / residual_out may alias.  */
ucclResult_t ucclAllReduceResidualRMSNorm(const void* x, const void* residual, const void* gamma,
                                          void* out, void* residualOut, int tokens, int hidden,
                                          float eps, ucclComm_t comm, void* stream);

/* Local GEMM on tcgen05: C[M,N] = A[M,K] * B[N,K]^T, bf16 in/out, fp32 accumulate.
 * epilogue 0: plain.  epilogue 1 (SwiGLU): B = [gate rows (N/2); up rows (N/2)],
 * C[M,N/2] = silu(A*gate^T) * (A*up^T).  No communicator needed. */
ucclResult_t ucclGemmBf16(const void* A, const void* B, void* C, int M, int N, int K, int lda,
                          int ldb, int ldc, int epilogue, void* stream);

/* all-gather -> GEMM: xShard [M/nranks, K] of every rank is gathered into the symmetric
 * scratch xFull [M, K] while C[M,N(/2)] = xFull * W[N,K]^T is computed in arrival order.
 * xFull must come from ucclMemAlloc. */
ucclResult_t ucclAllGatherGemm(const void* xShard, void* xFull, const void* W, void* C, int M,
                               int N, int K, int epilogue, ucclComm_t comm, void* stream);

/* GEMM -> reduce-scatter: partial = A[M,K] * W[N,K]^T lands in the symmetric scratch cPartial
 * [M, N]; out [M/nranks, N] receives the sum over ranks of this rank's row shard.
 * cPartial must come from ucclMemAlloc. */
ucclResult_t ucclGemmReduceScatter(const void* A, const void* W, void* cPartial, void* out, int M,
                                   int N, int K, ucclComm_t comm, void* stream);

/* MoE expert-parallel all-to-all (experts are spread evenly: rank r owns experts
 * [r * E / nranks, (r + 1) * E / nranks)).
 *
 * Dispatch sends every (token, k) pair to the rank that owns expert topkIdx[token][k]: the row is
 * converted from bf16 to fp8 e4m3 with one fp32 scale per 128 elements on the way.  Each source
 * rank owns a fixed region of `rowsPerSource` rows on every destination, so the receive area is
 * [nranks][rowsPerSource] rows and recvCounts[s] tells how many rows of region s are valid.
 * The caller runs its experts on the received rows and writes one bf16 output row per received
 * row, at the same index, into `expertOut`.  Combine then pulls, for every local token, its topk
 * output rows from the ranks that produced them and writes out = sum_k weight[k] * row_k. */
typedef struct ucclMoeContext* ucclMoeContext_t;
typedef struct {
  void* recvX;          /* fp8 e4m3 [nranks][rowsPerSource][hidden]                     */
  float* recvScale;     /* fp32     [nranks][rowsPerSource][hidden / 128]               */
  int32_t* recvMeta;    /* int32    [nranks][rowsPerSource][4]: source token, local expert, k, 1 */
  int32_t* recvCounts;  /* int32    [nranks] valid rows per source region               */
  void* expertOut;      /* bf16     [nranks][rowsPerSource][hidden], written by the caller */
  int rowsPerSource;
  int nranks;
} ucclMoeLayout_t;
/* Collective.  capacityFactor <= 0 sizes the regions for the worst case
 * (maxTokensPerRank * min(topk, numExperts / nranks) rows per source); a positive factor sizes
 * them to factor * maxTokensPerRank * topk / nranks rows and rows beyond that are dropped and
 * counted (ucclMoeOverflow). */
ucclResult_t ucclMoeCreate(ucclMoeContext_t* ctx, int maxTokensPerRank, int hidden, int numExperts, int topk,
                           float capacityFactor, ucclComm_t comm);
ucclResult_t ucclMoeDestroy(ucclMoeContext_t ctx);
ucclResult_t ucclMoeGetLayout(ucclMoeContext_t ctx, ucclMoeLayout_t* layout);
/* x [tokens, hidden] bf16, topkIdx [tokens, topk] int32 global expert ids (negative = unused). */
ucclResult_t ucclMoeDispatch(ucclMoeContext_t ctx, const void* x, const int32_t* topkIdx, int tokens, void* stream);
/* topkWeight [tokens, topk] fp32; out [tokens, hidden] bf16.  Uses the routing of the last dispatch. */
ucclResult_t ucclMoeCombine(ucclMoeContext_t ctx, const float* topkWeight, int tokens, void* out, void* stream);
/* Rows dropped so far because a region was full (always 0 with capacityFactor <= 0). */
ucclResult_t ucclMoeOverflow(ucclMoeContext_t ctx, unsigned int* rows);

/* ==================================================================
 * extensions: tuning, introspection, counters
 * ================================================================== */
typedef struct {
  int rank, nranks, nnodes, localRank, localRanks;
  int cudaDevice;     /* -1 on the CPU backend                      */
  int nChannels;
  int nvlsSupported;  /* multicast objects bound for the arena       */
  int p2pMode;        /* 0 none, 1 cudaIpc, 2 VMM fd, 3 in-process   */
  int netActive;      /* proxy thread + plugin in use                */
  char netName[64];
  size_t stagingBytes;
} ucclCommInfo_t;
ucclResult_t ucclCommGetInfo(ucclComm_t comm, ucclCommInfo_t* info);

typedef struct {
  uint64_t ops[8];          /* indexed by ucclCollKind_t                */
  uint64_t bytes[8];
  uint64_t algoHist[ucclNumAlgos];
  uint64_t proxyPosts, proxyCompletions, proxyHeartbeat;
  uint64_t waitTimeouts;
} ucclCounters_t;
typedef enum {
  ucclCollAllReduce = 0, ucclCollAllGather = 1, ucclCollReduceScatter = 2, ucclCollBroadcast = 3,
  ucclCollReduce = 4, ucclCollAllToAll = 5, ucclCollSendRecv = 6, ucclCollRma = 7
} ucclCollKind_t;
ucclResult_t ucclCommGetCounters(ucclComm_t comm, ucclCounters_t* counters);

/* Which algorithm/protocol/CTA count the tuner picks for (collective, bytes). */
ucclResult_t ucclCommQueryTuning(ucclComm_t comm, ucclCollKind_t coll, size_t bytes,
                                 int symmetric, ucclAlgo_t* algo, ucclProto_t* proto,
                                 int* nChannels);
/* Load a measured bus-bandwidth table (JSON written by the sweep benchmark). */
ucclResult_t ucclCommLoadTuning(ucclComm_t comm, const char* jsonPath);
/* Force algorithm/protocol for subsequent calls on this communicator (Auto = tuner). */
ucclResult_t ucclCommSetAlgo(ucclComm_t comm, ucclAlgo_t algo, ucclProto_t proto);
/* Force the number of CTAs ("channels") of subsequent collective kernels; 0 returns to the tuner. */
ucclResult_t ucclCommSetBlocks(ucclComm_t comm, int blocks);
/* Options of the fused all-gather -> GEMM on this communicator; 0 keeps the default of a field.
 * agMode: 1 = copy engines move the rows, 2 = communication CTAs inside the GEMM launch,
 *         3 = a forwarder warp in every GEMM CTA ("spread").
 * commCtas: number of those CTAs (mode 2); in mode 1 the number of copy-engine lanes (0 = one stream
 * per peer, k = k streams that serve the peers one after the other, nearest first).
 * ceChunks: copies per peer (mode 1).
 * The environment variables UCCL_FUSED_AG / UCCL_FUSED_COMM_CTAS / UCCL_FUSED_CE_CHUNKS win. */
ucclResult_t ucclCommSetFusedOptions(ucclComm_t comm, int agMode, int commCtas, int ceChunks);
/* The fused GEMM -> reduce-scatter has one transport: the epilogue TMA-stores every tile into the
 * owner's memory.  Its option: CTAs of the launch that do nothing but sum the staged partial tiles of
 * this rank's rows while the others compute (0 = none: every CTA computes, then sums; at most 64).
 * Worth it where the links rather than the tensor cores set the pace.  UCCL_FUSED_RS_REDUCERS wins. */
ucclResult_t ucclCommSetFusedRsReducers(ucclComm_t comm, int reducerCtas);
/* Fused all-reduce + residual + RMSNorm on the switch path: 1..4 = the kernel first all-reduces the rows
 * (that many rows of every CTA per pass), then normalises all rows from local memory; 0 = one phase,
 * every rank normalises the rows it reduced from registers and multicasts both results; -1 = default (1).
 * UCCL_NORM_MC_ROWS wins. */
ucclResult_t ucclCommSetFusedNormRows(ucclComm_t comm, int rows);

#ifdef __cplusplus
}
#endif
#endif /* UCCL_PUBLIC_H_ */
