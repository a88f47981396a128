// Ring all-reduce / all-gather / reduce-scatter over NVLink peer memory, Simple and LL128
// protocols.  One CTA = one channel; channel b moves slice b of every chunk.
//
// Schedule and primitives follow the reference's ring (src/algorithms/ring.cc:23-79 all-reduce,
// :299-325 all-gather, :386-415 reduce-scatter; src/device/primitives.hpp:31-179 send /
// recvReduceSend / recvReduceCopySend / recvCopySend), whose send and receive halves are
// placeholders.  Here they are real:
//   Simple : the sender stores a piece into a slot of the successor's step buffer, fences, and
//            advances the successor's tail counter; the receiver waits on its tail, consumes the
//            slot and advances the predecessor's head counter (credit).
//   LL128  : pieces travel as 128-byte lines whose words 7 and 15 carry the step sequence number;
//            a warp writes four lines with one 16-byte store per lane and the receiver's warp
//            polls until all four flag pairs match, so no separate tail write or fence is needed.
//            Credits still flow through the head counter.
// The NVSwitch makes every GPU a neighbour at full bandwidth, so the ring order is only a
// convention here; the algorithm is kept for parity and as the fallback when neither staging
// nor multicast is wanted.
#include "../host/ring_schedule.h"
#include "coll_device.cuh"
#include "collectives.cuh"

namespace uccl {
namespace dev {

constexpr int kLLLineBytes = 128;
constexpr int kLLDataPerLine = 112;

struct RingChan {
  const DevComm* dc;
  RingCtrl* mine;       // my control block for this channel
  RingCtrl* nextCtrl;   // successor's (I write its tail)
  RingCtrl* prevCtrl;   // predecessor's (I write its head)
  char* sendSlots;      // successor's slot array for this channel
  const char* recvSlots;  // my slot array for this channel
  size_t slotBytes;     // payload capacity of one slot
  uint64_t sent, rcvd;
  int next, prev;
  int proto;
};

__device__ __forceinline__ bool chan_wait_credit(RingChan& ch) {
  __shared__ int ok;
  if (threadIdx.x == 0)
    ok = ch.sent + 1 > kRingSlots
             ? wait_u64(&ch.mine->head, ch.sent + 1 - kRingSlots, *ch.dc, DEV_TIMEOUT_P2P, ch.next, static_cast<uint32_t>(ch.sent))
             : 1;
  __syncthreads();
  const bool r = ok != 0;
  __syncthreads();
  return r;
}
__device__ __forceinline__ bool chan_wait_data(RingChan& ch) {
  __shared__ int ok;
  if (threadIdx.x == 0)
    ok = wait_u64(&ch.mine->tail, ch.rcvd + 1, *ch.dc, DEV_TIMEOUT_P2P, ch.prev, static_cast<uint32_t>(ch.rcvd));
  __syncthreads();
  const bool r = ok != 0;
  __syncthreads();
  return r;
}
__device__ __forceinline__ void chan_post_send(RingChan& ch) {
  __syncthreads();
  ++ch.sent;
  if (threadIdx.x == 0 && ch.proto == ucclProtoSimple) {
    ptx::fence_sys();
    ptx::st_release_sys_u64(&ch.nextCtrl->tail, ch.sent);
  }
}
__device__ __forceinline__ void chan_post_recv(RingChan& ch) {
  __syncthreads();
  ++ch.rcvd;
  if (threadIdx.x == 0) {
    ptx::fence_sys();
    ptx::st_release_sys_u64(&ch.prevCtrl->head, ch.rcvd);
  }
}

// ---- element-wise piece operations (pieces are small enough for this to be latency bound) ----
template <int DT>
__device__ __forceinline__ void piece_sum(char* dst, const char* a, const char* b, size_t bytes) {
  using V = Vec<DT>;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | bytes) & 15) == 0) {
    for (size_t i = static_cast<size_t>(threadIdx.x) << 4; i < bytes; i += static_cast<size_t>(blockDim.x) << 4) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      V::add(acc, ptx::ld_global_v4(a + i));
      V::add(acc, ptx::ld_global_v4(b + i));
      ptx::st_global_v4(dst + i, V::pack(acc));
    }
  } else {
    const size_t n = bytes / V::ES;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x)
      V::store1(dst + i * V::ES, V::load1(a + i * V::ES) + V::load1(b + i * V::ES));
  }
}

// ---- LL128 line codec on the device: lane j of each group of 8 owns 16 bytes of a line ----
// data word index (0..13) carried in the first / second 8 bytes of lane j, or -1 for a flag
__device__ __forceinline__ int ll_word0(int j) { return j < 4 ? 2 * j : 2 * j - 1; }
__device__ __forceinline__ int ll_word1(int j) { return (j == 3 || j == 7) ? -1 : (j < 4 ? 2 * j + 1 : 2 * j); }

__device__ __forceinline__ uint64_t load_word(const char* src, size_t off, size_t bytes) {
  // 8 payload bytes at `off`, zero beyond `bytes`
  if (off + 8 <= bytes && ((reinterpret_cast<uintptr_t>(src) + off) & 7) == 0) return *reinterpret_cast<const uint64_t*>(src + off);
  uint64_t v = 0;
  for (int k = 0; k < 8; ++k)
    if (off + k < bytes) v |= static_cast<uint64_t>(static_cast<unsigned char>(src[off + k])) << (8 * k);
  return v;
}
__device__ __forceinline__ void store_word(char* dst, size_t off, size_t bytes, uint64_t v) {
  if (off + 8 <= bytes && ((reinterpret_cast<uintptr_t>(dst) + off) & 7) == 0) {
    *reinterpret_cast<uint64_t*>(dst + off) = v;
    return;
  }
  for (int k = 0; k < 8; ++k)
    if (off + k < bytes) dst[off + k] = static_cast<char>(v >> (8 * k));
}

// Write `bytes` of payload from src as LL128 lines into `slot` with sequence number seq.
__device__ __forceinline__ void ll128_send(char* slot, const char* src, size_t bytes, uint64_t seq) {
  const size_t lines = (bytes + kLLDataPerLine - 1) / kLLDataPerLine;
  for (size_t unit = threadIdx.x; unit < lines * 8; unit += blockDim.x) {
    const size_t line = unit >> 3;
    const int j = static_cast<int>(unit & 7);
    const int w0 = ll_word0(j), w1 = ll_word1(j);
    const uint64_t a = load_word(src, line * kLLDataPerLine + w0 * 8, bytes);
    const uint64_t b = w1 < 0 ? seq : load_word(src, line * kLLDataPerLine + w1 * 8, bytes);
    asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(slot + line * kLLLineBytes + j * 16), "l"(a), "l"(b) : "memory");
  }
}

// Wait for the lines of a piece and hand every payload word to `sink(byteOffset, word)`.
template <typename Sink>
__device__ __forceinline__ bool ll128_recv(const char* slot, size_t bytes, uint64_t seq, const DevComm& dc, int peer,
                                           Sink sink) {
  const size_t lines = (bytes + kLLDataPerLine - 1) / kLLDataPerLine;
  const uint64_t t0 = ptx::globaltimer_ns();
  bool ok = true;
  for (size_t unit = threadIdx.x; unit < lines * 8 && ok; unit += blockDim.x) {
    const size_t line = unit >> 3;
    const int j = static_cast<int>(unit & 7);
    const char* lp = slot + line * kLLLineBytes;
    // the line is complete when both flag words carry seq
    uint32_t spins = 0;
    while (true) {
      uint64_t f0, d0, f1, d1;
      asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(d0), "=l"(f0) : "l"(lp + 3 * 16) : "memory");
      asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(d1), "=l"(f1) : "l"(lp + 7 * 16) : "memory");
      if (f0 == seq && f1 == seq) break;
      if ((++spins & 63u) == 0) {
        if (aborted(dc)) { ok = false; break; }
        if (ptx::globaltimer_ns() - t0 > dc.timeoutNs) {
          record_status(dc, DEV_TIMEOUT_LL, peer, static_cast<uint32_t>(seq));
          ok = false;
          break;
        }
      }
    }
    if (!ok) break;
    uint64_t a, b;
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(lp + j * 16) : "memory");
    const int w0 = ll_word0(j), w1 = ll_word1(j);
    sink(line * kLLDataPerLine + w0 * 8, a);
    if (w1 >= 0) sink(line * kLLDataPerLine + w1 * 8, b);
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

template <int DT>
__device__ __forceinline__ uint64_t word_sum(uint64_t x, uint64_t y) {
  using V = Vec<DT>;
  if (DT == DT_F32) {
    const float a0 = __uint_as_float(static_cast<uint32_t>(x)) + __uint_as_float(static_cast<uint32_t>(y));
    const float a1 = __uint_as_float(static_cast<uint32_t>(x >> 32)) + __uint_as_float(static_cast<uint32_t>(y >> 32));
    return static_cast<uint64_t>(__float_as_uint(a0)) | (static_cast<uint64_t>(__float_as_uint(a1)) << 32);
  }
  uint32_t out[2];
  for (int h = 0; h < 2; ++h) {
    const uint32_t xa = static_cast<uint32_t>(x >> (32 * h)), ya = static_cast<uint32_t>(y >> (32 * h));
    if (DT == DT_BF16) {
      const float2 p = ptx::unpack_bf16x2(xa), q = ptx::unpack_bf16x2(ya);
      out[h] = ptx::pack_bf16x2(p.x + q.x, p.y + q.y);
    } else {
      const float2 p = ptx::unpack_f16x2(xa), q = ptx::unpack_f16x2(ya);
      out[h] = ptx::pack_f16x2(p.x + q.x, p.y + q.y);
    }
  }
  (void)sizeof(V);
  return static_cast<uint64_t>(out[0]) | (static_cast<uint64_t>(out[1]) << 32);
}

// ---- the three primitives every ring step is made of ----
enum RecvMode : int { RECV_NONE = 0, RECV_COPY = 1, RECV_SUM = 2, RECV_SUM_SEND = 3 };

// Moves one step of the ring: sends `sendBytes` from sendSrc (unless null), and receives
// `recvBytes`: COPY -> recvDst = incoming; SUM -> recvDst = addend + incoming;
// SUM_SEND -> successor gets addend + incoming (nothing is stored locally).
template <int DT>
__device__ bool ring_step(RingChan& ch, const char* sendSrc, size_t sendBytes, int recvMode, char* recvDst,
                          const char* addend, size_t recvBytes) {
  const size_t piece = ch.slotBytes;
  const size_t nS = sendSrc ? (sendBytes + piece - 1) / piece : 0;
  const size_t nR = recvMode != RECV_NONE ? (recvBytes + piece - 1) / piece : 0;
  const size_t nIter = nS > nR ? nS : nR;
  for (size_t j = 0; j < nIter; ++j) {
    if (j < nS) {
      const size_t off = j * piece, nb = min(piece, sendBytes - off);
      if (!chan_wait_credit(ch)) return false;
      char* slot = ch.sendSlots + (ch.sent % kRingSlots) * (ch.proto == ucclProtoLL128 ? size_t(kRingLLLines) * kLLLineBytes : piece);
      if (ch.proto == ucclProtoLL128) ll128_send(slot, sendSrc + off, nb, ch.sent + 1);
      else block_copy(slot, sendSrc + off, nb);
      chan_post_send(ch);
    }
    if (j < nR) {
      const size_t off = j * piece, nb = min(piece, recvBytes - off);
      const char* slot = ch.recvSlots + (ch.rcvd % kRingSlots) * (ch.proto == ucclProtoLL128 ? size_t(kRingLLLines) * kLLLineBytes : piece);
      char* out = nullptr;
      if (recvMode == RECV_SUM_SEND) {
        if (!chan_wait_credit(ch)) return false;
        out = ch.sendSlots + (ch.sent % kRingSlots) * (ch.proto == ucclProtoLL128 ? size_t(kRingLLLines) * kLLLineBytes : piece);
      }
      if (ch.proto == ucclProtoLL128) {
        const uint64_t seq = ch.rcvd + 1;
        bool ok;
        if (recvMode == RECV_COPY) {
          char* d = recvDst + off;
          ok = ll128_recv(slot, nb, seq, *ch.dc, ch.prev, [&](size_t o, uint64_t w) { store_word(d, o, nb, w); });
        } else if (recvMode == RECV_SUM) {
          char* d = recvDst + off;
          const char* ad = addend + off;
          ok = ll128_recv(slot, nb, seq, *ch.dc, ch.prev,
                          [&](size_t o, uint64_t w) { store_word(d, o, nb, word_sum<DT>(load_word(ad, o, nb), w)); });
        } else {
          // forward the sum as fresh LL128 lines: lane layout is identical on both sides
          const char* ad = addend + off;
          const uint64_t outSeq = ch.sent + 1;
          const size_t lines = (nb + kLLDataPerLine - 1) / kLLDataPerLine;
          ok = ll128_recv(slot, nb, seq, *ch.dc, ch.prev, [&](size_t o, uint64_t w) {
            const size_t line = o / kLLDataPerLine;
            const int word = static_cast<int>((o - line * kLLDataPerLine) >> 3);
            const int physical = word < 7 ? word : word + 1;  // skip flag word 7
            *reinterpret_cast<volatile uint64_t*>(out + line * kLLLineBytes + physical * 8) =
                word_sum<DT>(load_word(ad, o, nb), w);
          });
          if (ok) {
            // data words first, then the two flags of every line
            __syncthreads();
            ptx::fence_sys();
            for (size_t l = threadIdx.x; l < lines; l += blockDim.x) {
              *reinterpret_cast<volatile uint64_t*>(out + l * kLLLineBytes + 7 * 8) = outSeq;
              *reinterpret_cast<volatile uint64_t*>(out + l * kLLLineBytes + 15 * 8) = outSeq;
            }
          }
        }
        if (!ok) return false;
      } else {
        if (!chan_wait_data(ch)) return false;
        if (recvMode == RECV_COPY) block_copy(recvDst + off, slot, nb);
        else if (recvMode == RECV_SUM) piece_sum<DT>(recvDst + off, addend + off, slot, nb);
        else piece_sum<DT>(out, addend + off, slot, nb);
      }
      if (recvMode == RECV_SUM_SEND) chan_post_send(ch);
      chan_post_recv(ch);
    }
  }
  return true;
}

template <int DT>
__global__ void __launch_bounds__(kThreads, 1) ring_kernel(const __grid_constant__ RingArgs a) {
  using V = Vec<DT>;
  const DevComm& dc = a.dc;
  const int b = blockIdx.x, B = gridDim.x, n = dc.nranks, pos = a.ringPos;
  RingChan ch;
  ch.dc = &dc;
  ch.proto = a.proto;
  ch.next = a.ringNext;
  ch.prev = a.ringPrev;
  ch.mine = reinterpret_cast<RingCtrl*>(dc.arena[dc.rank] + kArenaRingCtrlOff) + b;
  ch.nextCtrl = reinterpret_cast<RingCtrl*>(dc.arena[a.ringNext] + kArenaRingCtrlOff) + b;
  ch.prevCtrl = reinterpret_cast<RingCtrl*>(dc.arena[a.ringPrev] + kArenaRingCtrlOff) + b;
  if (a.proto == ucclProtoLL128) {
    const size_t chanOff = kArenaRingLLOff + static_cast<size_t>(b) * kRingSlots * kRingLLLines * kLLLineBytes;
    ch.sendSlots = dc.arena[a.ringNext] + chanOff;
    ch.recvSlots = dc.arena[dc.rank] + chanOff;
    ch.slotBytes = static_cast<size_t>(kRingLLLines) * kLLDataPerLine;
  } else {
    const size_t chanBytes = (a.ringBufBytes / B) & ~size_t(kRingSlots * 16 - 1);
    ch.sendSlots = dc.arena[a.ringNext] + a.ringBufOff + static_cast<size_t>(b) * chanBytes;
    ch.recvSlots = dc.arena[dc.rank] + a.ringBufOff + static_cast<size_t>(b) * chanBytes;
    ch.slotBytes = chanBytes / kRingSlots;
  }
  ch.sent = ch.mine->sent;
  ch.rcvd = ch.mine->rcvd;

  const char* in = a.inUser;
  char* out = a.outUser;
  bool ok = true;
  if (a.coll == ucclCollAllReduce) {
    // slice b of the message, then n chunks of that slice
    size_t so, sl;
    split(a.count, B, b, &so, &sl);
    in += so * V::ES;
    out += so * V::ES;
    auto chunk = [&](int c, size_t* off, size_t* len) {
      ringChunk(sl, n, c, off, len);
      *off *= V::ES;
      *len *= V::ES;
    };
    for (int s = 0; s < n - 1 && ok; ++s) {
      size_t o1, l1, o2, l2;
      chunk(ringRsSendChunk(pos, s, n), &o1, &l1);
      chunk(ringRsRecvChunk(pos, s, n), &o2, &l2);
      ok = ring_step<DT>(ch, (s == 0 ? in : out) + o1, l1, RECV_SUM, out + o2, in + o2, l2);
    }
    for (int s = 0; s < n - 1 && ok; ++s) {
      size_t o1, l1, o2, l2;
      chunk(ringAgSendChunk(pos, s, n), &o1, &l1);
      chunk(ringAgRecvChunk(pos, s, n), &o2, &l2);
      ok = ring_step<DT>(ch, out + o1, l1, RECV_COPY, out + o2, nullptr, l2);
    }
  } else if (a.coll == ucclCollAllGather) {
    // chunk p (rank p's contribution) lives at out + p * count; channel b moves slice b of it
    size_t so, sl;
    split(a.count, B, b, &so, &sl);
    const size_t chunkStride = a.count * V::ES, off = so * V::ES, len = sl * V::ES;
    const int me = a.ringRanks[pos];
    if (out + me * chunkStride != in) block_copy(out + me * chunkStride + off, in + off, len);
    __syncthreads();
    for (int s = 0; s < n - 1 && ok; ++s) {
      const int sc = a.ringRanks[((pos - s) % n + n) % n], rc = a.ringRanks[((pos - s - 1) % n + n) % n];
      ok = ring_step<DT>(ch, (s == 0 ? in : out + sc * chunkStride) + off, len, RECV_COPY, out + rc * chunkStride + off,
                         nullptr, len);
    }
  } else {
    // reduce-scatter: the partial sum of a chunk hops around the ring and gains one term per hop.
    // Step 0 only sends, steps 1..n-2 receive + add + forward, step n-1 receives + adds into the
    // output.  The slice is cut into rounds of one piece per chunk, so that the send-only first
    // step never needs more than one free slot and the pieces travel in the order the successor
    // consumes them.
    size_t so, sl;
    split(a.count, B, b, &so, &sl);
    const size_t chunkStride = a.count * V::ES, off = so * V::ES, len = sl * V::ES;
    const size_t piece = ch.slotBytes;
    for (size_t ro = 0; ro < len && ok; ro += piece) {
      const size_t nb = min(piece, len - ro);
      const int c0 = a.ringRanks[((pos - 1) % n + n) % n];
      ok = ring_step<DT>(ch, in + c0 * chunkStride + off + ro, nb, RECV_NONE, nullptr, nullptr, 0);
      for (int k = 1; k < n && ok; ++k) {
        const int rc = a.ringRanks[((pos - 1 - k) % n + n) % n];
        const bool last = k == n - 1;
        ok = ring_step<DT>(ch, nullptr, 0, last ? RECV_SUM : RECV_SUM_SEND, out + off + ro,
                           in + rc * chunkStride + off + ro, nb);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    ch.mine->sent = ch.sent;
    ch.mine->rcvd = ch.rcvd;
  }
}

}  // namespace dev

cudaError_t launchRingKernel(const RingArgs& a, int blocks, cudaStream_t stream) {
  if (blocks < 1 || blocks > kMaxBlocks) return cudaErrorInvalidValue;
  if (a.proto == ucclProtoLL128 && blocks > kLLBlocks) return cudaErrorInvalidValue;
  switch (a.dtype) {
    case DEVDT_F16: dev::ring_kernel<dev::DT_F16><<<blocks, dev::kThreads, 0, stream>>>(a); break;
    case DEVDT_BF16: dev::ring_kernel<dev::DT_BF16><<<blocks, dev::kThreads, 0, stream>>>(a); break;
    case DEVDT_F32: dev::ring_kernel<dev::DT_F32><<<blocks, dev::kThreads, 0, stream>>>(a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace uccl
