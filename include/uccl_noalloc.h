/*
 * uccl_noalloc.h -- an entry point that never allocates memory.
 *
 * This entry point has no counterpart in the reference project.
 *
 * Who it is for: code that runs where calling the CUDA allocator is off the table -- a plugin
 * called from inside somebody else's memory pool, a real-time serving loop that must not take
 * the allocator's lock, a host that has already handed every byte of device memory to its own
 * arena.  The regular MoE dispatch needs a context object whose creation allocates counters, a
 * routing table and a receive area; callers like the above cannot create one.
 *
 * What it does: the single-GPU form of the MoE dispatch cast-and-route step.  Every (token, k)
 * pair of x is converted from bf16 to fp8 e4m3 with one fp32 scale per 128 elements and written,
 * together with its scales and a {token, expert, k, 1} descriptor, to the next free row of the
 * caller's output buffers; *recvCount receives the number of rows written.  Row order is not
 * deterministic (rows are claimed with an atomic counter).
 *
 * The kernel's bookkeeping (row counter, CTA completion counter, per-pair row table) lives in a
 * fixed array inside the library: UCCL_NOALLOC_SCRATCH_BYTES bytes on every GPU that loads the
 * library, held until the process exits.  Consequences the caller must know:
 *   - sizes are capped: tokens <= UCCL_NOALLOC_MAX_TOKENS, topk <= UCCL_NOALLOC_MAX_TOPK,
 *     hidden a multiple of 128 and <= 8192, rowsCapacity >= tokens * topk; anything else is
 *     refused with ucclInvalidArgument and a message in ucclNoAllocLastError();
 *   - all calls on one GPU share that array.  Each call clears what it needs at its start, in
 *     stream order, but two calls that can overlap on the GPU (different streams, no ordering
 *     between them) race on it;
 *   - the first call on each device looks up the array's device address; make that first call
 *     outside any stream capture.
 * No cudaMalloc, cudaFree or other allocating routine is called, on the first call or later.
 */
#ifndef UCCL_NOALLOC_H_
#define UCCL_NOALLOC_H_

#include "uccl.h"

#ifdef __cplusplus
extern "C" {
#endif

#define UCCL_NOALLOC_MAX_TOKENS 4096
#define UCCL_NOALLOC_MAX_TOPK 16
#define UCCL_NOALLOC_SCRATCH_BYTES (1024 + UCCL_NOALLOC_MAX_TOKENS * UCCL_NOALLOC_MAX_TOPK * 4)

/* x [tokens, hidden] bf16; topkIdx [tokens, topk] int32 (negative = unused slot);
 * recvX fp8 [rowsCapacity, hidden]; recvScale fp32 [rowsCapacity, hidden / 128];
 * recvMeta int32 [rowsCapacity, 4]; recvCount int32 [1].  All device pointers, 16-byte aligned. */
ucclResult_t ucclMoeDispatchLocalNoAlloc(const void* x, const int32_t* topkIdx, int tokens, int hidden, int numExperts,
                                         int topk, void* recvX, float* recvScale, int32_t* recvMeta, int32_t* recvCount,
                                         int rowsCapacity, void* stream);

/* Message of the last refusal or CUDA failure on the calling thread ("" if none). */
const char* ucclNoAllocLastError(void);

#ifdef __cplusplus
}
#endif
#endif /* UCCL_NOALLOC_H_ */
