// Point-to-point send / receive over NVLink: the sender copies into slots of the receiver's
// arena and bumps a tail counter there; the receiver drains the slots into the user's buffer and
// bumps a head counter in the sender's arena.  One launch carries a whole group of operations;
// every operation is striped over kP2pStripes CTAs, each with its own slice of the slots and its
// own pair of counters, so eight copy loops run in parallel per direction.
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

__global__ void __launch_bounds__(kThreads, 1) p2p_kernel(const __grid_constant__ P2pArgs a) {
  const DevComm& dc = a.dc;
  const int opIdx = blockIdx.x / kP2pStripes, stripe = blockIdx.x % kP2pStripes;
  if (opIdx >= a.nops) return;
  const P2pOp& op = a.ops[opIdx];
  // stripe split in 16-byte units; the last stripe carries the byte tail
  size_t off, len;
  {
    size_t o, l;
    split(op.bytes >> 4, kP2pStripes, stripe, &o, &l);
    off = o << 4;
    len = l << 4;
    if (stripe == kP2pStripes - 1) len += op.bytes & 15;
  }
  if (len == 0) return;
  __shared__ int s_ok;
  P2pCtrl* mine = ctrl_of(dc, dc.rank, op.peer, stripe);
  P2pCtrl* theirs = ctrl_of(dc, op.peer, dc.rank, stripe);
  if (op.isSend) {
    uint64_t sent = mine->sent;
    for (size_t done = 0; done < len; done += kStripeSlotBytes) {
      const size_t n = min(kStripeSlotBytes, len - done);
      if (threadIdx.x == 0)
        s_ok = wait_u64(&mine->head, sent + 1 >= kP2pSlots ? sent + 1 - kP2pSlots : 0, dc, DEV_TIMEOUT_P2P, op.peer,
                        static_cast<uint32_t>(sent));
      __syncthreads();
      if (!s_ok) return;
      block_copy(slot_of(dc, op.peer, dc.rank, static_cast<int>(sent % kP2pSlots), stripe), op.src + off + done, n);
      __syncthreads();
      ++sent;
      if (threadIdx.x == 0) {
        ptx::fence_sys();
        ptx::st_release_sys_u64(&theirs->tail, sent);
      }
    }
    if (threadIdx.x == 0) mine->sent = sent;
  } else {
    uint64_t rcvd = mine->rcvd;
    for (size_t done = 0; done < len; done += kStripeSlotBytes) {
      const size_t n = min(kStripeSlotBytes, len - done);
      if (threadIdx.x == 0) s_ok = wait_u64(&mine->tail, rcvd + 1, dc, DEV_TIMEOUT_P2P, op.peer, static_cast<uint32_t>(rcvd));
      __syncthreads();
      if (!s_ok) return;
      block_copy(op.dst + off + done, slot_of(dc, dc.rank, op.peer, static_cast<int>(rcvd % kP2pSlots), stripe), n);
      __syncthreads();
      ++rcvd;
      if (threadIdx.x == 0) {
        ptx::fence_sys();
        ptx::st_release_sys_u64(&theirs->head, rcvd);
      }
    }
    if (threadIdx.x == 0) mine->rcvd = rcvd;
  }
}

}  // namespace dev

cudaError_t launchP2pKernel(const P2pArgs& a, cudaStream_t stream) {
  if (a.nops < 1 || a.nops > kMaxP2pOps) return cudaErrorInvalidValue;
  dev::p2p_kernel<<<a.nops * kP2pStripes, dev::kThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace uccl
