// NVLink-domain collectives as single persistent kernels: one-shot, two-shot, NVLS (multimem)
// and low-latency all-reduce; pull / push all-gather; pull reduce-scatter; broadcast; reduce;
// all-to-all.
//
// Mapping to the reference: one-shot replaces src/algorithms/one_shot.cc:21-88, the symmetric
// pull kernels replace src/algorithms/symmetric.cc:23-278 (which have no cross-rank
// synchronisation and make every work-group redo the whole buffer), "channels" are the CTAs of
// one launch instead of one single-work-group launch per channel (src/enqueue.cc:216-231), and
// sums are carried in fp32 (the reference adds in the 16-bit type, src/device/reduce_kernel.hpp:19).
//
// Common shape of every kernel:
//   [copy user input into the local work buffer]  -> rank barrier (peers' inputs are ready)
//   -> remote loads / stores / multimem ops        -> rank barrier (peers are done with my memory)
//   -> [copy the local work buffer out to the user's buffer]
// Work buffers are 16-byte aligned and padded to whole 16-byte vectors by the host side, so the
// inner loops only ever move uint4.
#include "collectives.cuh"

#include "coll_device.cuh"

namespace uccl {
namespace dev {

// slice `b` of `B` of the byte range [0, bytes), in whole 16-byte vectors (bytes % 16 == 0)
__device__ __forceinline__ void slice16(size_t bytes, int B, int b, size_t* off, size_t* len) {
  size_t o, l;
  split(bytes >> 4, B, b, &o, &l);
  *off = o << 4;
  *len = l << 4;
}
// slice of an arbitrary byte range: vectors are spread over CTAs, the last CTA takes the tail
__device__ __forceinline__ void slice_bytes(size_t bytes, int B, int b, size_t* off, size_t* len) {
  slice16(bytes & ~size_t(15), B, b, off, len);
  if (b == B - 1) *len += bytes & 15;
}

// copy [begin, begin+len) of a padded range, but never past the exact user length
__device__ __forceinline__ void copy_clamped(char* dstBase, const char* srcBase, size_t begin, size_t len,
                                             size_t userBytes) {
  if (begin >= userBytes) return;
  block_copy(dstBase + begin, srcBase + begin, min(len, userBytes - begin));
}

template <int DT>
__device__ __forceinline__ uint4 reduce_peers(const CollArgs& a, size_t byteOff) {
  using V = Vec<DT>;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int n = a.dc.nranks;
  uint4 v[UCCL_MAX_LOCAL_RANKS > 8 ? 8 : UCCL_MAX_LOCAL_RANKS];
  for (int p0 = 0; p0 < n; p0 += 8) {
    const int m = min(8, n - p0);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < m) v[j] = ptx::ld_stream_v4(a.in[(a.dc.rank + p0 + j) % n] + byteOff);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < m) V::add(acc, v[j]);
  }
  return V::pack(acc);
}

// U vectors `stride` bytes apart from NP ranks each, all NP * U loads issued before the first add.
// With two or four ranks a single vector per step leaves only two or four 16-byte loads in flight
// per thread, far too few to cover the NVLink latency; callers pick U so that NP * U = 8.
template <int DT, int U, int NP>
__device__ __forceinline__ void reduce_peers_fixed(const CollArgs& a, size_t byteOff, size_t stride, uint4 (&out)[U]) {
  using V = Vec<DT>;
  uint4 v[U][NP];
#pragma unroll
  for (int j = 0; j < U; ++j)
#pragma unroll
    for (int p = 0; p < NP; ++p) v[j][p] = ptx::ld_stream_v4(a.in[(a.dc.rank + p) % NP] + byteOff + j * stride);
#pragma unroll
  for (int j = 0; j < U; ++j) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int p = 0; p < NP; ++p) V::add(acc, v[j][p]);
    out[j] = V::pack(acc);
  }
}

// out(i) for every 16-byte vector i in [begin, end) handled by this thread, with `sink(i, vector)`
template <int DT, typename Sink>
__device__ __forceinline__ void reduce_range(const CollArgs& a, size_t srcBase, size_t begin, size_t end, Sink sink) {
  const size_t stride = static_cast<size_t>(blockDim.x) << 4;
  const int n = a.dc.nranks;
  size_t i = begin + (static_cast<size_t>(threadIdx.x) << 4);
  if (n == 2) {
    for (; i + 3 * stride < end; i += 4 * stride) {
      uint4 o[4];
      reduce_peers_fixed<DT, 4, 2>(a, srcBase + i, stride, o);
#pragma unroll
      for (int j = 0; j < 4; ++j) sink(i + j * stride, o[j]);
    }
  } else if (n == 4) {
    for (; i + stride < end; i += 2 * stride) {
      uint4 o[2];
      reduce_peers_fixed<DT, 2, 4>(a, srcBase + i, stride, o);
#pragma unroll
      for (int j = 0; j < 2; ++j) sink(i + j * stride, o[j]);
    }
  }
  for (; i < end; i += stride) sink(i, reduce_peers<DT>(a, srcBase + i));
}

// ------------------------------------------------------------------ all-reduce, one-shot
template <int DT>
__device__ void ar_oneshot(const CollArgs& a) {
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x;
  size_t off, len;
  slice16(a.bytes, B, b, &off, &len);
  if (a.inUser) copy_clamped(const_cast<char*>(a.in[dc.rank]), a.inUser, off, len, a.userBytes);
  if (!rank_barrier(dc)) return;
  char* dst = a.out[dc.rank];
  reduce_range<DT>(a, 0, off, off + len, [&](size_t i, uint4 v) { st_out16(dst + i, v); });
  if (!rank_barrier(dc)) return;
  if (a.outUser) copy_clamped(a.outUser, dst, off, len, a.userBytes);
}

// ------------------------------------------------------------------ all-reduce, two-shot / NVLS
// Block b owns slice b of every rank's shard for the copies, and slice b of its own rank's
// shard for the reduction, so that the CTA-level barrier with CTA b of each peer covers exactly
// the data it depends on.
template <int DT, bool NVLS>
__device__ void ar_twoshot(const CollArgs& a) {
  using V = Vec<DT>;
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x, n = dc.nranks;
  const size_t nvec = a.bytes >> 4;
  if (a.inUser) {
    for (int s = 0; s < n; ++s) {
      size_t so, sl, o, l;
      split(nvec, n, s, &so, &sl);
      split(sl, B, b, &o, &l);
      copy_clamped(const_cast<char*>(a.in[dc.rank]), a.inUser, (so + o) << 4, l << 4, a.userBytes);
    }
  }
  if (!rank_barrier(dc)) return;
  {
    size_t so, sl, o, l;
    split(nvec, n, dc.rank, &so, &sl);
    split(sl, B, b, &o, &l);
    const size_t begin = (so + o) << 4, end = (so + o + l) << 4;
    const size_t stride = static_cast<size_t>(blockDim.x) << 4;
    if (NVLS) {
      size_t i = begin + (static_cast<size_t>(threadIdx.x) << 4);
      for (; i + 3 * stride < end; i += 4 * stride) {
        const uint4 v0 = V::mc_reduce(a.inMc + i);
        const uint4 v1 = V::mc_reduce(a.inMc + i + stride);
        const uint4 v2 = V::mc_reduce(a.inMc + i + 2 * stride);
        const uint4 v3 = V::mc_reduce(a.inMc + i + 3 * stride);
        ptx::multimem_st_v4(a.outMc + i, v0);
        ptx::multimem_st_v4(a.outMc + i + stride, v1);
        ptx::multimem_st_v4(a.outMc + i + 2 * stride, v2);
        ptx::multimem_st_v4(a.outMc + i + 3 * stride, v3);
      }
      for (; i < end; i += stride) ptx::multimem_st_v4(a.outMc + i, V::mc_reduce(a.inMc + i));
    } else {
      reduce_range<DT>(a, 0, begin, end, [&](size_t i, uint4 v) {
        for (int p = 0; p < n; ++p) ptx::st_global_v4(a.out[(dc.rank + p) % n] + i, v);
      });
    }
  }
  if (!rank_barrier(dc)) return;
  if (a.outUser) {
    for (int s = 0; s < n; ++s) {
      size_t so, sl, o, l;
      split(nvec, n, s, &so, &sl);
      split(sl, B, b, &o, &l);
      copy_clamped(a.outUser, a.out[dc.rank], (so + o) << 4, l << 4, a.userBytes);
    }
  }
}

// ------------------------------------------------------------------ all-reduce, low latency
// Every rank stores its data into a dedicated slot of every peer's arena as 16-byte packets
// {data0, flag, data1, flag}; a packet is valid once both flags equal the CTA's epoch.  No barrier
// and no prior knowledge of the peers' buffers is needed: one NVLink traversal end to end.
// CTA b handles bytes [b * kLLDataPerBlock, ...).  Slots are double-buffered by epoch parity: a
// rank can be at most one operation ahead of a peer, because finishing an operation requires
// every peer's packets of that same operation.
template <int DT>
__device__ void ar_ll(const CollArgs& a) {
  using V = Vec<DT>;
  const DevComm& dc = a.dc;
  const int b = blockIdx.x, n = dc.nranks, t = threadIdx.x;
  const uint32_t e = dc.llEpochs[b] + 1;
  const int parity = e & 1;
  const size_t base = static_cast<size_t>(b) * kLLDataPerBlock;
  const size_t valid = a.bytes > base ? min(static_cast<size_t>(kLLDataPerBlock), a.bytes - base) : 0;
  const size_t unitOff = static_cast<size_t>(t) * 8;  // this thread's 8 data bytes
  constexpr int EPU = 8 / V::ES;                      // elements per unit
  float mine[EPU];
  int nel = 0;
  if (unitOff < valid) {
    nel = static_cast<int>(min(static_cast<size_t>(8), valid - unitOff) / V::ES);
    for (int j = 0; j < EPU; ++j) mine[j] = j < nel ? V::load1(a.inUser + base + unitOff + j * V::ES) : 0.f;
    // pack my elements into two 32-bit words
    uint32_t w0, w1;
    if (DT == DT_F32) {
      w0 = __float_as_uint(mine[0]);
      w1 = __float_as_uint(mine[EPU - 1]);
    } else if (DT == DT_BF16) {
      w0 = ptx::pack_bf16x2(mine[0], mine[1 % EPU]);
      w1 = ptx::pack_bf16x2(mine[2 % EPU], mine[3 % EPU]);
    } else {
      w0 = ptx::pack_f16x2(mine[0], mine[1 % EPU]);
      w1 = ptx::pack_f16x2(mine[2 % EPU], mine[3 % EPU]);
    }
    const uint4 pkt = make_uint4(w0, e, w1, e);
    const size_t slotOff = kArenaLLOff +
                           ((static_cast<size_t>(parity) * kLLBlocks + b) * UCCL_MAX_LOCAL_RANKS + dc.rank) * kLLSlotBytes +
                           static_cast<size_t>(t) * 16;
    for (int p = 1; p < n; ++p) ptx::st_volatile_v4(dc.arena[(dc.rank + p) % n] + slotOff, pkt);
  }
  bool ok = true;
  if (unitOff < valid) {
    float acc[EPU];
    for (int j = 0; j < EPU; ++j) acc[j] = mine[j];
    const uint64_t t0 = ptx::globaltimer_ns();
    for (int p = 1; p < n && ok; ++p) {
      const int peer = (dc.rank + p) % n;
      const char* slot = dc.arena[dc.rank] + kArenaLLOff +
                         ((static_cast<size_t>(parity) * kLLBlocks + b) * UCCL_MAX_LOCAL_RANKS + peer) * kLLSlotBytes +
                         static_cast<size_t>(t) * 16;
      uint4 pkt;
      uint32_t spins = 0;
      while (true) {
        pkt = ptx::ld_volatile_v4(slot);
        if (pkt.y == e && pkt.w == e) break;
        if ((++spins & 63u) == 0) {
          if (aborted(dc)) { ok = false; break; }
          if (ptx::globaltimer_ns() - t0 > dc.timeoutNs) {
            record_status(dc, DEV_TIMEOUT_LL, peer, e);
            ok = false;
            break;
          }
        }
      }
      if (!ok) break;
      if (DT == DT_F32) {
        acc[0] += __uint_as_float(pkt.x);
        acc[EPU - 1] += (EPU > 1) ? __uint_as_float(pkt.z) : 0.f;
      } else if (DT == DT_BF16) {
        const float2 f0 = ptx::unpack_bf16x2(pkt.x), f1 = ptx::unpack_bf16x2(pkt.z);
        acc[0] += f0.x; acc[1 % EPU] += f0.y; acc[2 % EPU] += f1.x; acc[3 % EPU] += f1.y;
      } else {
        const float2 f0 = ptx::unpack_f16x2(pkt.x), f1 = ptx::unpack_f16x2(pkt.z);
        acc[0] += f0.x; acc[1 % EPU] += f0.y; acc[2 % EPU] += f1.x; acc[3 % EPU] += f1.y;
      }
    }
    if (ok)
      for (int j = 0; j < nel; ++j) V::store1(a.outUser + base + unitOff + j * V::ES, acc[j]);
  }
  __syncthreads();
  if (t == 0) dc.llEpochs[b] = e;
}

// ------------------------------------------------------------------ all-gather / reduce-scatter, low latency
// The packet scheme of ar_ll for the two chunked collectives, same slots and epochs: a.bytes is the
// size of one rank's chunk (at most kLLBlocks * kLLDataPerBlock), CTA b and thread t own the same
// 8 bytes of every chunk.
//   reduce-scatter: the unit of chunk p goes to rank p; a rank adds the n - 1 units it receives to
//                   its own (fp32) and stores the result.
//   all-gather:     the unit of my chunk goes to every peer; a rank stores the n - 1 units it
//                   receives next to its own.  Bytes only, no element type.
//   all-to-all:     the unit of chunk p goes to rank p, which stores it as chunk [sender] of its output.
// Every rank sends to every peer and waits for every peer in both, so the rule that makes the
// double-buffered slots safe holds as for the all-reduce: nobody can be more than one operation ahead.
__device__ __forceinline__ void ll_load_unit(const char* p, int nbytes, uint32_t& w0, uint32_t& w1) {
  if (nbytes == 8 && (reinterpret_cast<uintptr_t>(p) & 7) == 0) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    w0 = v.x;
    w1 = v.y;
    return;
  }
  uint32_t w[2] = {0u, 0u};
  for (int j = 0; j < nbytes; ++j) w[j >> 2] |= static_cast<uint32_t>(static_cast<unsigned char>(p[j])) << (8 * (j & 3));
  w0 = w[0];
  w1 = w[1];
}
__device__ __forceinline__ void ll_store_unit(char* p, int nbytes, uint32_t w0, uint32_t w1) {
  if (nbytes == 8 && (reinterpret_cast<uintptr_t>(p) & 7) == 0) {
    *reinterpret_cast<uint2*>(p) = make_uint2(w0, w1);
    return;
  }
  const uint32_t w[2] = {w0, w1};
  for (int j = 0; j < nbytes; ++j) p[j] = static_cast<char>(w[j >> 2] >> (8 * (j & 3)));
}
template <int DT>
__device__ __forceinline__ void ll_accumulate(float (&acc)[4], uint32_t w0, uint32_t w1) {
  if (DT == DT_F32) {
    acc[0] += __uint_as_float(w0);
    acc[1] += __uint_as_float(w1);
  } else if (DT == DT_BF16) {
    const float2 f0 = ptx::unpack_bf16x2(w0), f1 = ptx::unpack_bf16x2(w1);
    acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
  } else {
    const float2 f0 = ptx::unpack_f16x2(w0), f1 = ptx::unpack_f16x2(w1);
    acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
  }
}
// waits for the packet of epoch e in `slot`; false on abort or when the time is up
__device__ __forceinline__ bool ll_wait_packet(const DevComm& dc, const char* slot, uint32_t e, int peer, uint64_t t0, uint4* pkt) {
  uint32_t spins = 0;
  while (true) {
    *pkt = ptx::ld_volatile_v4(slot);
    if (pkt->y == e && pkt->w == e) return true;
    if ((++spins & 63u) == 0) {
      if (aborted(dc)) return false;
      if (ptx::globaltimer_ns() - t0 > dc.timeoutNs) {
        record_status(dc, DEV_TIMEOUT_LL, peer, e);
        return false;
      }
    }
  }
}

enum : int { LL_REDUCE_SCATTER = 0, LL_ALLGATHER = 1, LL_ALLTOALL = 2 };
template <int DT, int MODE>
__device__ void chunk_ll(const CollArgs& a) {
  constexpr bool GATHER = MODE == LL_ALLGATHER;
  constexpr bool REDUCE = MODE == LL_REDUCE_SCATTER;
  const DevComm& dc = a.dc;
  const int b = blockIdx.x, n = dc.nranks, t = threadIdx.x, me = dc.rank;
  const uint32_t e = dc.llEpochs[b] + 1;
  const int parity = e & 1;
  const size_t base = static_cast<size_t>(b) * kLLDataPerBlock;
  const size_t valid = a.bytes > base ? min(static_cast<size_t>(kLLDataPerBlock), a.bytes - base) : 0;
  const size_t unitOff = static_cast<size_t>(t) * 8;
  if (unitOff < valid) {
    const int nb = static_cast<int>(min(static_cast<size_t>(8), valid - unitOff));
    const size_t off = base + unitOff;
    const size_t slotBase = kArenaLLOff + (static_cast<size_t>(parity) * kLLBlocks + b) * UCCL_MAX_LOCAL_RANKS * kLLSlotBytes +
                            static_cast<size_t>(t) * 16;
    // send
    uint32_t m0, m1;  // my own unit: of my chunk (gather) or of chunk `me` of my input (reduce-scatter, all-to-all)
    if (GATHER) {
      ll_load_unit(a.inUser + off, nb, m0, m1);
      const uint4 pkt = make_uint4(m0, e, m1, e);
      for (int q = 1; q < n; ++q)
        ptx::st_volatile_v4(dc.arena[(me + q) % n] + slotBase + static_cast<size_t>(me) * kLLSlotBytes, pkt);
    } else {
      for (int q = 1; q < n; ++q) {
        const int p = (me + q) % n;
        uint32_t w0, w1;
        ll_load_unit(a.inUser + static_cast<size_t>(p) * a.inStride + off, nb, w0, w1);
        ptx::st_volatile_v4(dc.arena[p] + slotBase + static_cast<size_t>(me) * kLLSlotBytes, make_uint4(w0, e, w1, e));
      }
      ll_load_unit(a.inUser + static_cast<size_t>(me) * a.inStride + off, nb, m0, m1);
    }
    // receive
    const uint64_t t0 = ptx::globaltimer_ns();
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (REDUCE) {
      ll_accumulate<DT>(acc, m0, m1);
    } else {
      char* own = a.outUser + static_cast<size_t>(me) * a.outStride + off;
      if (own != a.inUser + (GATHER ? 0 : static_cast<size_t>(me) * a.inStride) + off) ll_store_unit(own, nb, m0, m1);
    }
    bool ok = true;
    for (int q = 1; q < n && ok; ++q) {
      const int p = (me + q) % n;
      uint4 pkt;
      ok = ll_wait_packet(dc, dc.arena[me] + slotBase + static_cast<size_t>(p) * kLLSlotBytes, e, p, t0, &pkt);
      if (!ok) break;
      if (REDUCE) ll_accumulate<DT>(acc, pkt.x, pkt.z);
      else ll_store_unit(a.outUser + static_cast<size_t>(p) * a.outStride + off, nb, pkt.x, pkt.z);
    }
    if (ok && REDUCE) {
      uint32_t w0, w1;
      if (DT == DT_F32) {
        w0 = __float_as_uint(acc[0]);
        w1 = __float_as_uint(acc[1]);
      } else if (DT == DT_BF16) {
        w0 = ptx::pack_bf16x2(acc[0], acc[1]);
        w1 = ptx::pack_bf16x2(acc[2], acc[3]);
      } else {
        w0 = ptx::pack_f16x2(acc[0], acc[1]);
        w1 = ptx::pack_f16x2(acc[2], acc[3]);
      }
      ll_store_unit(a.outUser + off, nb, w0, w1);
    }
  }
  __syncthreads();
  if (t == 0) dc.llEpochs[b] = e;
}

// ------------------------------------------------------------------ all-gather
// pull: every rank reads each peer's chunk straight into its own output
__device__ void ag_pull(const CollArgs& a) {
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x, n = dc.nranks;
  size_t off, len;
  slice_bytes(a.chunkBytes, B, b, &off, &len);
  if (a.inUser) block_copy(const_cast<char*>(a.in[dc.rank]) + off, a.inUser + off, len);
  if (!rank_barrier(dc)) return;
  for (int p = 0; p < n; ++p) {
    const int peer = (dc.rank + p) % n;
    block_copy(a.outUser + static_cast<size_t>(peer) * a.outStride + off, a.in[peer] + off, len);
  }
  rank_barrier(dc);
}

// push: every rank writes its chunk into slot [rank] of each peer's output (multimem.st
// reaches all of them with one store when the output has a multicast alias)
__device__ void ag_push(const CollArgs& a) {
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x, n = dc.nranks;
  size_t off, len;
  slice16(a.chunkBytes, B, b, &off, &len);
  if (!rank_barrier(dc)) return;  // peers are done with the previous contents of their output
  const size_t dstOff = static_cast<size_t>(dc.rank) * a.outStride;
  const size_t stride = static_cast<size_t>(blockDim.x) << 4;
  if (a.outMc) {
    size_t i = off + (static_cast<size_t>(threadIdx.x) << 4);
    for (; i + 3 * stride < off + len; i += 4 * stride) {
      const uint4 v0 = ptx::ld_global_v4(a.inUser + i), v1 = ptx::ld_global_v4(a.inUser + i + stride);
      const uint4 v2 = ptx::ld_global_v4(a.inUser + i + 2 * stride), v3 = ptx::ld_global_v4(a.inUser + i + 3 * stride);
      ptx::multimem_st_v4(a.outMc + dstOff + i, v0);
      ptx::multimem_st_v4(a.outMc + dstOff + i + stride, v1);
      ptx::multimem_st_v4(a.outMc + dstOff + i + 2 * stride, v2);
      ptx::multimem_st_v4(a.outMc + dstOff + i + 3 * stride, v3);
    }
    for (; i < off + len; i += stride) ptx::multimem_st_v4(a.outMc + dstOff + i, ptx::ld_global_v4(a.inUser + i));
  } else {
    for (size_t i = off + (static_cast<size_t>(threadIdx.x) << 4); i < off + len; i += stride) {
      const uint4 v = ptx::ld_global_v4(a.inUser + i);
      for (int p = 0; p < n; ++p) ptx::st_global_v4(a.out[(dc.rank + p) % n] + dstOff + i, v);
    }
  }
  rank_barrier(dc);
}

// ------------------------------------------------------------------ reduce-scatter (pull)
template <int DT>
__device__ void rs_pull(const CollArgs& a) {
  using V = Vec<DT>;
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x, n = dc.nranks;
  size_t off, len;
  slice16(a.chunkBytes, B, b, &off, &len);  // chunkBytes is padded to 16 by the host
  if (a.inUser) {
    // user chunks are inStride apart and exactly userBytes long; staged chunks are chunkBytes apart
    for (int s = 0; s < n; ++s)
      copy_clamped(const_cast<char*>(a.in[dc.rank]) + static_cast<size_t>(s) * a.chunkBytes,
                   a.inUser + static_cast<size_t>(s) * a.inStride, off, len, a.userBytes);
  }
  if (!rank_barrier(dc)) return;
  // inside the work buffers chunk s starts at s * workStride
  const size_t workStride = a.inUser ? a.chunkBytes : a.inStride;
  const size_t src = static_cast<size_t>(dc.rank) * workStride;
  char* dst = a.out[dc.rank];
  const size_t stride = static_cast<size_t>(blockDim.x) << 4;
  if (a.inMc) {
    size_t i = off + (static_cast<size_t>(threadIdx.x) << 4);
    for (; i + 7 * stride < off + len; i += 8 * stride) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = V::mc_reduce(a.inMc + src + i + j * stride);
#pragma unroll
      for (int j = 0; j < 8; ++j) st_out16(dst + i + j * stride, v[j]);
    }
    for (; i + 3 * stride < off + len; i += 4 * stride) {
      const uint4 v0 = V::mc_reduce(a.inMc + src + i), v1 = V::mc_reduce(a.inMc + src + i + stride);
      const uint4 v2 = V::mc_reduce(a.inMc + src + i + 2 * stride), v3 = V::mc_reduce(a.inMc + src + i + 3 * stride);
      st_out16(dst + i, v0);
      st_out16(dst + i + stride, v1);
      st_out16(dst + i + 2 * stride, v2);
      st_out16(dst + i + 3 * stride, v3);
    }
    for (; i < off + len; i += stride) st_out16(dst + i, V::mc_reduce(a.inMc + src + i));
  } else {
    reduce_range<DT>(a, src, off, off + len, [&](size_t i, uint4 v) { st_out16(dst + i, v); });
  }
  if (!rank_barrier(dc)) return;
  if (a.outUser) copy_clamped(a.outUser, dst, off, len, a.userBytes);
}

// ------------------------------------------------------------------ broadcast
// pull: the root exposes its data (in place if symmetric, else through its staging area) and
// every other rank copies it out with plain loads
__device__ void bcast_pull(const CollArgs& a) {
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x;
  size_t off, len;
  slice_bytes(a.userBytes, B, b, &off, &len);
  const bool isRoot = dc.rank == a.root;
  if (isRoot && a.inUser) block_copy(const_cast<char*>(a.in[dc.rank]) + off, a.inUser + off, len);
  if (!rank_barrier(dc)) return;
  if (!isRoot) {
    block_copy(a.outUser + off, a.in[a.root] + off, len);
  } else {
    const char* src = a.inUser ? a.inUser : a.in[dc.rank];
    if (a.outUser != src) block_copy(a.outUser + off, src + off, len);
  }
  rank_barrier(dc);
}

__device__ void bcast_push(const CollArgs& a) {
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x, n = dc.nranks;
  size_t off, len;
  slice16(a.bytes, B, b, &off, &len);
  if (!rank_barrier(dc)) return;
  if (dc.rank == a.root) {
    const size_t stride = static_cast<size_t>(blockDim.x) << 4;
    auto put = [&](size_t i, uint4 v) {
      if (a.outMc) {
        ptx::multimem_st_v4(a.outMc + i, v);
      } else {
        for (int p = 0; p < n; ++p) ptx::st_global_v4(a.out[(dc.rank + p) % n] + i, v);
      }
    };
    size_t i = off + (static_cast<size_t>(threadIdx.x) << 4);
    for (; i + 3 * stride < off + len; i += 4 * stride) {  // four loads in flight per thread
      const uint4 v0 = ptx::ld_global_v4(a.inUser + i), v1 = ptx::ld_global_v4(a.inUser + i + stride);
      const uint4 v2 = ptx::ld_global_v4(a.inUser + i + 2 * stride), v3 = ptx::ld_global_v4(a.inUser + i + 3 * stride);
      put(i, v0);
      put(i + stride, v1);
      put(i + 2 * stride, v2);
      put(i + 3 * stride, v3);
    }
    for (; i < off + len; i += stride) put(i, ptx::ld_global_v4(a.inUser + i));
  }
  rank_barrier(dc);
}

// ------------------------------------------------------------------ reduce (pull at the root)
template <int DT>
__device__ void reduce_pull(const CollArgs& a) {
  using V = Vec<DT>;
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x;
  size_t off, len;
  slice16(a.bytes, B, b, &off, &len);
  if (a.inUser) copy_clamped(const_cast<char*>(a.in[dc.rank]), a.inUser, off, len, a.userBytes);
  if (!rank_barrier(dc)) return;
  char* dst = a.out[dc.rank];
  if (dc.rank == a.root) {
    const size_t stride = static_cast<size_t>(blockDim.x) << 4;
    for (size_t i = off + (static_cast<size_t>(threadIdx.x) << 4); i < off + len; i += stride)
      st_out16(dst + i, a.inMc ? V::mc_reduce(a.inMc + i) : reduce_peers<DT>(a, i));
  }
  if (!rank_barrier(dc)) return;
  if (dc.rank == a.root && a.outUser) copy_clamped(a.outUser, dst, off, len, a.userBytes);
}

// ------------------------------------------------------------------ all-to-all (pull)
__device__ void a2a_pull(const CollArgs& a) {
  const DevComm& dc = a.dc;
  const int B = gridDim.x, b = blockIdx.x, n = dc.nranks;
  size_t off, len;
  slice_bytes(a.chunkBytes, B, b, &off, &len);
  const size_t workStride = a.inUser ? ((a.chunkBytes + 15) & ~size_t(15)) : a.inStride;
  if (a.inUser)
    for (int s = 0; s < n; ++s)
      block_copy(const_cast<char*>(a.in[dc.rank]) + static_cast<size_t>(s) * workStride + off,
                 a.inUser + static_cast<size_t>(s) * a.inStride + off, len);
  if (!rank_barrier(dc)) return;
  for (int p = 0; p < n; ++p) {
    const int peer = (dc.rank + p) % n;
    block_copy(a.outUser + static_cast<size_t>(peer) * a.outStride + off,
               a.in[peer] + static_cast<size_t>(dc.rank) * workStride + off, len);
  }
  rank_barrier(dc);
}

// ------------------------------------------------------------------ helpers of copy-engine mode
template <int DT>
__device__ void local_reduce(const CollArgs& a) {
  using V = Vec<DT>;
  const int B = gridDim.x, b = blockIdx.x, nslots = a.root;
  size_t off, len;
  slice16(a.bytes, B, b, &off, &len);
  const char* src = a.in[0];
  char* dst = a.out[0];
  const size_t stride = static_cast<size_t>(blockDim.x) << 4;
  for (size_t i = off + (static_cast<size_t>(threadIdx.x) << 4); i < off + len; i += stride) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < nslots; ++s) V::add(acc, ptx::ld_global_v4(src + static_cast<size_t>(s) * a.inStride + i));
    const uint4 v = V::pack(acc);
    if (i + 16 <= a.userBytes) {
      st_out16(dst + i, v);
    } else {
      // last, partial vector: element stores only
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      for (size_t k = 0; i + k < a.userBytes; k += 2)
        *reinterpret_cast<uint16_t*>(dst + i + k) = static_cast<uint16_t>(w[k >> 2] >> (8 * (k & 3)));
    }
  }
}

// ------------------------------------------------------------------ kernel entry
template <int K, int DT>
__global__ void __launch_bounds__(kThreads, 1) coll_kernel(const __grid_constant__ CollArgs a) {
  if (K == KERN_AR_ONESHOT) ar_oneshot<DT>(a);
  if (K == KERN_AR_TWOSHOT) ar_twoshot<DT, false>(a);
  if (K == KERN_AR_NVLS) ar_twoshot<DT, true>(a);
  if (K == KERN_AR_LL) ar_ll<DT>(a);
  if (K == KERN_RS_LL) chunk_ll<DT, LL_REDUCE_SCATTER>(a);
  if (K == KERN_AG_LL) chunk_ll<DT, LL_ALLGATHER>(a);
  if (K == KERN_A2A_LL) chunk_ll<DT, LL_ALLTOALL>(a);
  if (K == KERN_AG_PULL) ag_pull(a);
  if (K == KERN_AG_PUSH) ag_push(a);
  if (K == KERN_RS_PULL) rs_pull<DT>(a);
  if (K == KERN_BCAST_PULL) bcast_pull(a);
  if (K == KERN_BCAST_PUSH) bcast_push(a);
  if (K == KERN_REDUCE_PULL) reduce_pull<DT>(a);
  if (K == KERN_A2A_PULL) a2a_pull(a);
  if (K == KERN_BARRIER) rank_barrier(a.dc);
  if (K == KERN_LOCAL_REDUCE) local_reduce<DT>(a);
}

}  // namespace dev

template <int K>
static cudaError_t launchTyped(const CollArgs& a, int blocks, cudaStream_t stream) {
  switch (a.dtype) {
    case dev::DT_F16: dev::coll_kernel<K, dev::DT_F16><<<blocks, dev::kThreads, 0, stream>>>(a); break;
    case dev::DT_BF16: dev::coll_kernel<K, dev::DT_BF16><<<blocks, dev::kThreads, 0, stream>>>(a); break;
    case dev::DT_F32: dev::coll_kernel<K, dev::DT_F32><<<blocks, dev::kThreads, 0, stream>>>(a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}
template <int K>
static cudaError_t launchUntyped(const CollArgs& a, int blocks, cudaStream_t stream) {
  dev::coll_kernel<K, dev::DT_F32><<<blocks, dev::kThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launchCollKernel(CollKernel k, const CollArgs& a, int blocks, cudaStream_t stream) {
  if (blocks < 1 || blocks > kMaxBlocks) return cudaErrorInvalidValue;
  switch (k) {
    case KERN_AR_ONESHOT: return launchTyped<KERN_AR_ONESHOT>(a, blocks, stream);
    case KERN_AR_TWOSHOT: return launchTyped<KERN_AR_TWOSHOT>(a, blocks, stream);
    case KERN_AR_NVLS: return launchTyped<KERN_AR_NVLS>(a, blocks, stream);
    case KERN_AR_LL: return blocks <= kLLBlocks ? launchTyped<KERN_AR_LL>(a, blocks, stream) : cudaErrorInvalidValue;
    case KERN_AG_PULL: return launchUntyped<KERN_AG_PULL>(a, blocks, stream);
    case KERN_AG_PUSH: return launchUntyped<KERN_AG_PUSH>(a, blocks, stream);
    case KERN_RS_PULL: return launchTyped<KERN_RS_PULL>(a, blocks, stream);
    case KERN_BCAST_PULL: return launchUntyped<KERN_BCAST_PULL>(a, blocks, stream);
    case KERN_BCAST_PUSH: return launchUntyped<KERN_BCAST_PUSH>(a, blocks, stream);
    case KERN_REDUCE_PULL: return launchTyped<KERN_REDUCE_PULL>(a, blocks, stream);
    case KERN_A2A_PULL: return launchUntyped<KERN_A2A_PULL>(a, blocks, stream);
    case KERN_BARRIER: return launchUntyped<KERN_BARRIER>(a, 1, stream);
    case KERN_LOCAL_REDUCE: return launchTyped<KERN_LOCAL_REDUCE>(a, blocks, stream);
    case KERN_RS_LL: return blocks <= kLLBlocks ? launchTyped<KERN_RS_LL>(a, blocks, stream) : cudaErrorInvalidValue;
    case KERN_AG_LL: return blocks <= kLLBlocks ? launchUntyped<KERN_AG_LL>(a, blocks, stream) : cudaErrorInvalidValue;
    case KERN_A2A_LL: return blocks <= kLLBlocks ? launchUntyped<KERN_A2A_LL>(a, blocks, stream) : cudaErrorInvalidValue;
  }
  return cudaErrorInvalidValue;
}

}  // namespace uccl
