// Index algebra of the ring algorithms, shared by the host ring (CPU backend), the GPU ring
// kernels and the self tests.  The reference spells the same schedule inline in its kernels
// (src/algorithms/ring.cc:24-79: n-1 reduce-scatter steps followed by n-1 all-gather steps,
// chunk = count / n with the remainder folded into the last chunk); here the chunks are balanced
// (sizes differ by at most one element) and the formulas are checked against a brute-force
// simulator for every n in [1, 16].
#pragma once
#include <stddef.h>

#if defined(__CUDACC__)
#define UCCL_HD __host__ __device__ __forceinline__
#else
#define UCCL_HD inline
#endif

namespace uccl {

// Chunk `idx` of `count` elements split into `n` balanced chunks.
UCCL_HD void ringChunk(size_t count, int n, int idx, size_t* off, size_t* len) {
  const size_t base = count / static_cast<size_t>(n), rem = count % static_cast<size_t>(n);
  const size_t i = static_cast<size_t>(idx);
  *off = i * base + (i < rem ? i : rem);
  *len = base + (i < rem ? 1 : 0);
}

// All-reduce, reduce-scatter phase, step s in [0, n-1): rank r sends chunk (r - s) and receives
// (and accumulates) chunk (r - s - 1).  After the phase rank r owns the full sum of chunk r + 1.
UCCL_HD int ringRsSendChunk(int r, int s, int n) { return ((r - s) % n + n) % n; }
UCCL_HD int ringRsRecvChunk(int r, int s, int n) { return ((r - s - 1) % n + n) % n; }
// All-gather phase, step s in [0, n-1): rank r sends chunk (r + 1 - s) and receives chunk (r - s).
UCCL_HD int ringAgSendChunk(int r, int s, int n) { return ((r + 1 - s) % n + n) % n; }
UCCL_HD int ringAgRecvChunk(int r, int s, int n) { return ((r - s) % n + n) % n; }

}  // namespace uccl
