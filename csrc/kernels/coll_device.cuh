// Device-side building blocks of the NVLink collectives: bounded waits, the cross-rank CTA
// barrier on signal pads, typed 16-byte accumulate/pack helpers and balanced work splitting.
//
// These replace the reference's Primitives<T,RedOp,Proto> layer (src/device/primitives.hpp:31-179,
// whose send/recv are placeholders) and its reduce helpers (src/device/reduce_kernel.hpp:17-80,
// which accumulate in the 16-bit type): every sum here is carried in fp32, every peer access is a
// direct load/store on a peer-mapped pointer or a multimem instruction on the multicast alias,
// and every wait has a deadline after which the kernel records why it gave up and returns.
#pragma once
#include "coll_device_types.h"
#include "device_comm.h"
#include "ptx.cuh"

namespace uccl {
namespace dev {

constexpr int kThreads = 512;

enum : int { DT_F16 = DEVDT_F16, DT_BF16 = DEVDT_BF16, DT_F32 = DEVDT_F32 };

// ------------------------------------------------------------------ status + bounded waits
__device__ __forceinline__ void record_status(const DevComm& dc, uint32_t code, int peer, uint32_t step) {
  // mapped host memory, plain stores: the first writer wins well enough for a diagnostic
  if (dc.status && ptx::ld_relaxed_sys_u32(dc.status) == 0) {
    ptx::st_relaxed_sys_u32(dc.status + 1, static_cast<uint32_t>(dc.rank));
    ptx::st_relaxed_sys_u32(dc.status + 2, static_cast<uint32_t>(peer));
    ptx::st_relaxed_sys_u32(dc.status + 3, step);
    ptx::st_relaxed_sys_u32(dc.status + 4, blockIdx.x);
    ptx::fence_sys();
    ptx::st_relaxed_sys_u32(dc.status, code);
  }
}

__device__ __forceinline__ bool aborted(const DevComm& dc) {
  return dc.abortFlag && ptx::ld_relaxed_sys_u32(dc.abortFlag) != 0;
}

// Spins until (int)(*p - target) >= 0.  Gives up on abort or after dc.timeoutNs.
__device__ __forceinline__ bool wait_u32(const uint32_t* p, uint32_t target, const DevComm& dc, uint32_t code,
                                         int peer, uint32_t step) {
  // poll with relaxed loads and order the data behind the flag with one fence on success: an
  // acquire on every poll is a system-scope fence per iteration
  if (static_cast<int32_t>(ptx::ld_relaxed_sys_u32(p) - target) >= 0) {
    ptx::fence_sys();
    return true;
  }
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (static_cast<int32_t>(ptx::ld_relaxed_sys_u32(p) - target) >= 0) {
      ptx::fence_sys();
      return true;
    }
    if ((++spins & 31u) == 0) {
      if (aborted(dc)) return false;
      if (ptx::globaltimer_ns() - t0 > dc.timeoutNs) {
        record_status(dc, code, peer, step);
        return false;
      }
    }
    if (spins > 64) __nanosleep(100);  // a long wait stops competing with the traffic it waits for
  }
}
__device__ __forceinline__ bool wait_u64(const uint64_t* p, uint64_t target, const DevComm& dc, uint32_t code,
                                         int peer, uint32_t step) {
  if (ptx::ld_relaxed_sys_u64(p) >= target) {
    ptx::fence_sys();
    return true;
  }
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ptx::ld_relaxed_sys_u64(p) >= target) {
      ptx::fence_sys();
      return true;
    }
    if ((++spins & 31u) == 0) {
      if (aborted(dc)) return false;
      if (ptx::globaltimer_ns() - t0 > dc.timeoutNs) {
        record_status(dc, code, peer, step);
        return false;
      }
    }
    if (spins > 64) __nanosleep(100);  // a long wait stops competing with the traffic it waits for
  }
}

// ------------------------------------------------------------------ cross-rank CTA barrier
// CTA b of every rank meets CTA b of every other rank.  Each rank owns one 128-byte line per CTA
// in its arena, word r of which rank r writes; a barrier writes the CTA's next epoch into word
// [b][my rank] of every peer and waits until all words [b][*] of its own line reached it.
// Everything the CTA wrote before the barrier is visible to peers that passed it, and the
// other way round.  Returns false if a peer did not show up in time (all threads agree).
//
// One thread does it all: a system-scope fence costs about as much whether one thread of the
// CTA issues it or sixteen do, and with a fence, a release store and two more fences in each of
// nranks threads a 96-CTA launch spent more time in its barriers than in its data (measured at
// four ranks, 256 KiB all-reduce: 27 us with 4 CTAs, 134 us with 96).  Here: the CTA barrier
// orders every thread's writes before thread 0's fence, which orders them before its relaxed flag
// stores; the peers' words share a line and are polled with 16-byte loads, with a short pause
// between polls once the first few have missed.
__device__ __forceinline__ bool rank_barrier(const DevComm& dc) {
  __shared__ int s_ok;
  const int b = blockIdx.x;
  __syncthreads();
  if (threadIdx.x == 0) {
    const int n = dc.nranks, me = dc.rank;
    const uint32_t e = dc.epochs[b] + 1;
    ptx::fence_sys();
    for (int q = 1; q < n; ++q) {
      const int p = me + q < n ? me + q : me + q - n;
      ptx::st_relaxed_sys_u32(reinterpret_cast<uint32_t*>(dc.arena[p] + kArenaBarrierOff) + b * kBarrierSlotWords + me, e);
    }
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(dc.arena[me] + kArenaBarrierOff) + b * kBarrierSlotWords;
    bool ok = true;
    uint64_t t0 = 0;
    uint32_t spins = 0, pause = 0;
    while (true) {
      int missing = -1;
#pragma unroll
      for (int v = 0; v < UCCL_MAX_LOCAL_RANKS / 4; ++v) {
        if (4 * v < n) {
          const uint4 w = ptx::ld_relaxed_sys_v4(mine + 4 * v);
          const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int p = 4 * v + k;
            if (p < n && p != me && static_cast<int32_t>(ws[k] - e) < 0) missing = p;
          }
        }
      }
      if (missing < 0) break;
      if (spins++ == 0) t0 = ptx::globaltimer_ns();
      if ((spins & 31u) == 0) {
        if (aborted(dc)) {
          ok = false;
          break;
        }
        if (ptx::globaltimer_ns() - t0 > dc.timeoutNs) {
          record_status(dc, DEV_TIMEOUT_BARRIER, missing, e);
          ok = false;
          break;
        }
      }
      if (spins > 8) {
        pause = pause < 160 ? pause + 20 : 160;
        __nanosleep(pause);
      }
    }
    ptx::fence_sys();
    dc.epochs[b] = e;  // advance even on failure: peers did too
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// ------------------------------------------------------------------ typed helpers
template <int DT>
struct Vec;  // elements per 16 bytes and conversions

template <>
struct Vec<DT_BF16> {
  static constexpr int N = 8;
  static constexpr int ES = 2;
  __device__ static __forceinline__ void add(float (&a)[8], uint4 v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = ptx::unpack_bf16x2(w[j]);
      a[2 * j] += f.x;
      a[2 * j + 1] += f.y;
    }
  }
  __device__ static __forceinline__ uint4 pack(const float (&a)[8]) {
    return make_uint4(ptx::pack_bf16x2(a[0], a[1]), ptx::pack_bf16x2(a[2], a[3]), ptx::pack_bf16x2(a[4], a[5]),
                      ptx::pack_bf16x2(a[6], a[7]));
  }
  __device__ static __forceinline__ float load1(const void* p) { return __bfloat162float(*static_cast<const __nv_bfloat16*>(p)); }
  __device__ static __forceinline__ void store1(void* p, float f) { *static_cast<__nv_bfloat16*>(p) = __float2bfloat16(f); }
  __device__ static __forceinline__ uint4 mc_reduce(const void* mc) { return ptx::multimem_ld_reduce_bf16x8(mc); }
};
template <>
struct Vec<DT_F16> {
  static constexpr int N = 8;
  static constexpr int ES = 2;
  __device__ static __forceinline__ void add(float (&a)[8], uint4 v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = ptx::unpack_f16x2(w[j]);
      a[2 * j] += f.x;
      a[2 * j + 1] += f.y;
    }
  }
  __device__ static __forceinline__ uint4 pack(const float (&a)[8]) {
    return make_uint4(ptx::pack_f16x2(a[0], a[1]), ptx::pack_f16x2(a[2], a[3]), ptx::pack_f16x2(a[4], a[5]),
                      ptx::pack_f16x2(a[6], a[7]));
  }
  __device__ static __forceinline__ float load1(const void* p) { return __half2float(*static_cast<const __half*>(p)); }
  __device__ static __forceinline__ void store1(void* p, float f) { *static_cast<__half*>(p) = __float2half(f); }
  __device__ static __forceinline__ uint4 mc_reduce(const void* mc) { return ptx::multimem_ld_reduce_f16x8(mc); }
};
template <>
struct Vec<DT_F32> {
  static constexpr int N = 4;
  static constexpr int ES = 4;
  __device__ static __forceinline__ void add(float (&a)[8], uint4 v) {
    a[0] += __uint_as_float(v.x);
    a[1] += __uint_as_float(v.y);
    a[2] += __uint_as_float(v.z);
    a[3] += __uint_as_float(v.w);
  }
  __device__ static __forceinline__ uint4 pack(const float (&a)[8]) {
    return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3]));
  }
  __device__ static __forceinline__ float load1(const void* p) { return *static_cast<const float*>(p); }
  __device__ static __forceinline__ void store1(void* p, float f) { *static_cast<float*>(p) = f; }
  __device__ static __forceinline__ uint4 mc_reduce(const void* mc) { return ptx::multimem_ld_reduce_f32x4(mc); }
};

// Balanced split of `total` items into `parts`; part `idx` is [*off, *off + *len).
__device__ __forceinline__ void split(size_t total, int parts, int idx, size_t* off, size_t* len) {
  const size_t base = total / static_cast<size_t>(parts), rem = total % static_cast<size_t>(parts);
  const size_t i = static_cast<size_t>(idx);
  *off = i * base + (i < rem ? i : rem);
  *len = base + (i < rem ? 1 : 0);
}

// 16-byte store to a destination that is at least 2-byte aligned (local memory only).
__device__ __forceinline__ void st_out16(char* dst, uint4 v) {
  if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    ptx::st_global_v4(dst, v);
  } else if ((reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
    uint32_t* d = reinterpret_cast<uint32_t*>(dst);
    d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
  } else {
    uint16_t* d = reinterpret_cast<uint16_t*>(dst);
    d[0] = static_cast<uint16_t>(v.x); d[1] = static_cast<uint16_t>(v.x >> 16);
    d[2] = static_cast<uint16_t>(v.y); d[3] = static_cast<uint16_t>(v.y >> 16);
    d[4] = static_cast<uint16_t>(v.z); d[5] = static_cast<uint16_t>(v.z >> 16);
    d[6] = static_cast<uint16_t>(v.w); d[7] = static_cast<uint16_t>(v.w >> 16);
  }
}

template <typename T>
__device__ __forceinline__ void block_copy_as(char* dst, const char* src, size_t n) {
  const size_t cnt = n / sizeof(T);
  const T* s = reinterpret_cast<const T*>(src);
  T* d = reinterpret_cast<T*>(dst);
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) d[i] = s[i];
  // bytes that do not fill a T
  const size_t done = cnt * sizeof(T);
  for (size_t i = done + threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
}

// CTA-wide copy of n bytes with the widest access the two addresses allow.
__device__ __forceinline__ void block_copy(char* dst, const char* src, size_t n) {
  const uintptr_t al = reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src);
  if ((al & 15) == 0) {
    const size_t nv = n >> 4;
    size_t i = threadIdx.x;
    for (; i + 3 * blockDim.x < nv; i += 4 * blockDim.x) {
      const uint4 a = ptx::ld_global_v4(src + (i << 4));
      const uint4 b = ptx::ld_global_v4(src + ((i + blockDim.x) << 4));
      const uint4 c = ptx::ld_global_v4(src + ((i + 2 * blockDim.x) << 4));
      const uint4 d = ptx::ld_global_v4(src + ((i + 3 * blockDim.x) << 4));
      ptx::st_global_v4(dst + (i << 4), a);
      ptx::st_global_v4(dst + ((i + blockDim.x) << 4), b);
      ptx::st_global_v4(dst + ((i + 2 * blockDim.x) << 4), c);
      ptx::st_global_v4(dst + ((i + 3 * blockDim.x) << 4), d);
    }
    for (; i < nv; i += blockDim.x) ptx::st_global_v4(dst + (i << 4), ptx::ld_global_v4(src + (i << 4)));
    for (size_t j = (nv << 4) + threadIdx.x; j < n; j += blockDim.x) dst[j] = src[j];
  } else if ((al & 7) == 0) {
    block_copy_as<uint64_t>(dst, src, n);
  } else if ((al & 3) == 0) {
    block_copy_as<uint32_t>(dst, src, n);
  } else if ((al & 1) == 0) {
    block_copy_as<uint16_t>(dst, src, n);
  } else {
    block_copy_as<uint8_t>(dst, src, n);
  }
}

}  // namespace dev
}  // namespace uccl
