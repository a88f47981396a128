// Point-to-point send / receive over NVLink: the sender copies into slots of the receiver's
// arena and bumps a tail counter there; the receiver drains the slots into the user's buffer and
// bumps a head counter in the sender's arena.  One launch carries a whole group of operations;
// operations with the same peer and direction share a FIFO and run one after the other as a
// chain, different chains run side by side.  Every chain has kP2pStripes CTAs, each with its own
// slice of the slots and its own pair of counters; an operation uses p2pStripesFor(bytes) of them
// (one per 512 KiB), so up to 32 copy loops run in parallel per direction: one CTA moves only about
// 7 GB/s through its FIFO (copy, system-scope fence, flag, per 128 KiB slot), measured 57 GB/s for
// a 1 GiB message with eight.
//
// The reference lists send/recv as future work (desgin/design-spec.md:1760); its P2P transport
// stub copies into a local staging buffer that no peer ever opens (src/transport/p2p.cc:107-151).
#include "coll_device.cuh"
#include "collectives.cuh"

namespace uccl {
namespace dev {

constexpr size_t kStripeSlotBytes = kP2pSlotBytes / kP2pStripes;

__device__ __forceinline__ P2pCtrl* ctrl_of(const DevComm& dc, int owner, int peer, int stripe) {
  return reinterpret_cast<P2pCtrl*>(dc.arena[owner] + kArenaP2pCtrlOff) + peer * kP2pStripes + stripe;
}
// slot `slot` of the FIFO sender -> receiver, stripe `stripe`, inside the receiver's arena
__device__ __forceinline__ char* slot_of(const DevComm& dc, int receiver, int sender, int slot, int stripe) {
  return dc.arena[receiver] + kArenaP2pDataOff + (static_cast<size_t>(sender) * kP2pSlots + slot) * kP2pSlotBytes +
         static_cast<size_t>(stripe) * kStripeSlotBytes;
}

// CTA-wide copy with eight 16-byte loads in flight per thread (32 KiB per CTA): what limits a
// FIFO's rate is the number of bytes on their way across the link, and 32 CTAs with four loads each
// kept about a third of the 1.4 MB in flight that 700 GB/s at 2 us need (224 GB/s for 1 GiB).
__device__ __noinline__ void p2p_copy(char* dst, const char* src, size_t n) {
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) != 0) {
    block_copy(dst, src, n);
    return;
  }
  // pieces are at most 128 KiB: 32-bit offsets
  const uint32_t bytes = static_cast<uint32_t>(n) & ~15u, TB = blockDim.x << 4;
  uint32_t o = threadIdx.x << 4;
  for (; o + 7 * TB < bytes; o += 8 * TB) {
    uint4 v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = ptx::ld_global_v4(src + o + k * TB);
#pragma unroll
    for (int k = 0; k < 8; ++k) ptx::st_global_v4(dst + o + k * TB, v[k]);
  }
  for (; o < bytes; o += TB) ptx::st_global_v4(dst + o, ptx::ld_global_v4(src + o));
  for (uint32_t j = bytes + threadIdx.x; j < n; j += blockDim.x) dst[j] = src[j];
}

// 256 threads and at least four CTAs per SM: every CTA of a launch that has work must be resident,
// because it waits for its counterpart on the peer, which waits for this rank's other CTAs in turn
constexpr int kP2pThreads = 256;
__global__ void __launch_bounds__(kP2pThreads, 4) p2p_kernel(const __grid_constant__ P2pArgs a) {
  const DevComm& dc = a.dc;
  const int chain = blockIdx.x / kP2pStripes, stripe = blockIdx.x % kP2pStripes;
  if (chain >= a.nchains) return;
  __shared__ int s_ok;
  const int first = a.heads[chain];
  const int peer = a.ops[first].peer;
  const bool isSend = a.ops[first].isSend != 0;
  P2pCtrl* mine = ctrl_of(dc, dc.rank, peer, stripe);
  P2pCtrl* theirs = ctrl_of(dc, peer, dc.rank, stripe);
  // slots of this stripe's FIFO used so far; carried from one operation of the chain to the next
  uint64_t pos = isSend ? mine->sent : mine->rcvd;
  for (int oi = first; oi >= 0; oi = a.ops[oi].next) {
    const P2pOp& op = a.ops[oi];
    const int stripes = p2pStripesFor(op.bytes);
    if (stripe >= stripes) continue;  // this operation is too small to need this CTA
    // stripe split in 16-byte units; the last stripe carries the byte tail
    size_t off, len;
    {
      size_t o, l;
      split(op.bytes >> 4, stripes, stripe, &o, &l);
      off = o << 4;
      len = l << 4;
      if (stripe == stripes - 1) len += op.bytes & 15;
    }
    // a stripe's share travels in at least four pieces (32 KiB or more each, at most a slot), so
    // that the receiver drains one piece while the sender fills the next
    size_t piece = ((len + 3) / 4 + 15) & ~size_t(15);
    piece = min(kStripeSlotBytes, max(piece, static_cast<size_t>(32u << 10)));
    for (size_t done = 0; done < len; done += piece) {
      const size_t n = min(piece, len - done);
      if (isSend) {
        if (threadIdx.x == 0)
          s_ok = wait_u64(&mine->head, pos + 1 >= kP2pSlots ? pos + 1 - kP2pSlots : 0, dc, DEV_TIMEOUT_P2P, peer,
                          static_cast<uint32_t>(pos));
        __syncthreads();
        if (!s_ok) return;
        p2p_copy(slot_of(dc, peer, dc.rank, static_cast<int>(pos % kP2pSlots), stripe), op.src + off + done, n);
        __syncthreads();
        ++pos;
        // the release orders the CTA's copies (which the barrier above ordered before this thread) before the flag
        if (threadIdx.x == 0) ptx::st_release_sys_u64(&theirs->tail, pos);
      } else {
        if (threadIdx.x == 0) s_ok = wait_u64(&mine->tail, pos + 1, dc, DEV_TIMEOUT_P2P, peer, static_cast<uint32_t>(pos));
        __syncthreads();
        if (!s_ok) return;
        p2p_copy(op.dst + off + done, slot_of(dc, dc.rank, peer, static_cast<int>(pos % kP2pSlots), stripe), n);
        __syncthreads();
        ++pos;
        if (threadIdx.x == 0) ptx::st_release_sys_u64(&theirs->head, pos);
      }
    }
  }
  if (threadIdx.x == 0) {
    if (isSend) mine->sent = pos;
    else mine->rcvd = pos;
  }
}

}  // namespace dev

cudaError_t launchP2pKernel(const P2pArgs& a, cudaStream_t stream) {
  if (a.nchains < 1 || a.nchains > kMaxP2pChains) return cudaErrorInvalidValue;
  // the whole grid must fit the device at once (see kP2pThreads)
  static thread_local int capDev = -1, capacity = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != capDev) {
    int perSm = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, dev::p2p_kernel, dev::kP2pThreads, 0) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return cudaGetLastError();
    capacity = perSm * sms;
    capDev = dev;
  }
  if (a.nchains * kP2pStripes > capacity) return cudaErrorLaunchOutOfResources;
  dev::p2p_kernel<<<a.nchains * kP2pStripes, dev::kP2pThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace uccl
