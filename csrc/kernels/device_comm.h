// Device-visible view of a communicator, passed by value to every collective kernel.
// Plain C structs shared by host code and kernels.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "uccl.h"

namespace uccl {

constexpr int kMaxBlocks = 128;       // CTAs a collective kernel may use ("channels")
constexpr int kLLBlocks = 16;         // CTAs the low-latency protocol may use
constexpr int kLLDataPerBlock = 4096; // payload bytes per CTA per peer per LL operation
constexpr int kLLSlotBytes = 2 * kLLDataPerBlock;  // each 8 data bytes travel with 8 flag bytes
constexpr int kP2pSlots = 4;               // FIFO depth per stripe: four pieces in flight hide the credit round trip
constexpr size_t kP2pSlotBytes = 4u << 20;  // one slot of every stripe together (128 KiB per stripe)

// Arena layout (byte offsets inside every rank's symmetric arena).
constexpr size_t kArenaBarrierOff = 0;                 // u32 [kMaxBlocks][kBarrierSlotWords]: one 128-byte line per CTA, word r written by rank r
constexpr int kBarrierSlotWords = 32;
static_assert(UCCL_MAX_LOCAL_RANKS <= kBarrierSlotWords, "a CTA's barrier words must fit one line");
// fused GEMM flags: one 128-byte line per 128-row block (see FLAG_STRIDE in gemm_sm100.cuh)
constexpr size_t kGemmFlagStrideBytes = 128;
constexpr int kGemmMaxRowBlocks = 1024;
constexpr size_t kArenaGemmReadyOff = 512u << 10;      // all-gather arrival counters, 128 KiB
constexpr size_t kArenaGemmDoneOff = 768u << 10;       // reduce-scatter counters, 128 KiB
constexpr size_t kArenaP2pCtrlOff = 96u << 10;         // P2pCtrl [UCCL_MAX_LOCAL_RANKS][kP2pStripes]
constexpr size_t kArenaMoeCtrlOff = 128u << 10;        // MoE counters (see moe.cu)
constexpr size_t kArenaLLOff = 1u << 20;               // [2][kLLBlocks][UCCL_MAX_LOCAL_RANKS][kLLSlotBytes]
constexpr size_t kArenaLLBytes = 2ull * kLLBlocks * UCCL_MAX_LOCAL_RANKS * kLLSlotBytes;  // 4 MiB
// LL128 ring: per channel kRingSlots slots of kRingLLLines 128-byte lines, written by the ring
// predecessor.  The region is only ever written with LL128 lines, so a stale word can never be
// mistaken for a current flag.
constexpr int kRingSlots = 4;
constexpr int kRingLLLines = 64;                          // 64 lines = 8 KiB = 7168 payload bytes
constexpr size_t kArenaRingLLOff = kArenaLLOff + kArenaLLBytes;
constexpr size_t kArenaRingLLBytes = 1u << 20;            // [kLLBlocks][kRingSlots][kRingLLLines][128]
constexpr size_t kArenaP2pDataOff = kArenaRingLLOff + kArenaRingLLBytes;  // [nranks][kP2pSlots][kP2pSlotBytes]
constexpr size_t kArenaRingCtrlOff = 176u << 10;          // RingCtrl [kMaxBlocks]

// Flow control of one ring channel (CTA).  `tail` is written by the ring predecessor (slots it
// filled for me), `head` by the successor (slots of mine it drained); `sent` / `rcvd` are this
// rank's own running counts.  All count slots since communicator creation.
struct RingCtrl {
  uint64_t tail;
  uint64_t head;
  uint64_t sent;
  uint64_t rcvd;
  uint64_t pad[4];
};

// Control words of the point-to-point FIFOs between this rank and one peer, for one stripe; the
// arena holds P2pCtrl [UCCL_MAX_LOCAL_RANKS][kP2pStripes] indexed by peer.  All four counters
// count slots since communicator creation.
constexpr int kP2pStripes = 32;  // CTAs (and independent sub-FIFOs) a point-to-point operation may use
// Stripes an operation of `bytes` bytes is cut into: one per 512 KiB (four full slots), so that a
// small message costs one CTA and a large one gets them all; every piece that travels costs
// several microseconds of fence and flag latency, so thin stripes lose more than they gain
// (4 MiB: 51 us on 8 stripes, 77-89 us on 32).  Sender and receiver compute it from the same byte count.
#ifdef __CUDACC__
#define UCCL_HOST_DEVICE __host__ __device__
#else
#define UCCL_HOST_DEVICE
#endif
inline UCCL_HOST_DEVICE int p2pStripesFor(size_t bytes) {
  const size_t s = bytes >> 19;
  return s < 1 ? 1 : (s > static_cast<size_t>(kP2pStripes) ? kP2pStripes : static_cast<int>(s));
}
struct P2pCtrl {
  uint64_t tail;  // written remotely by the peer when it is the sender: slots it has filled for me
  uint64_t head;  // written remotely by the peer when it is the receiver: slots of mine it has drained
  uint64_t sent;  // local: slots I have filled for the peer
  uint64_t rcvd;  // local: slots from the peer I have drained
  uint64_t pad[4];
};

struct DevComm {
  int rank;    // index inside the NVLink domain
  int nranks;  // size of the NVLink domain
  char* arena[UCCL_MAX_LOCAL_RANKS];  // every rank's arena, peer-mapped; arena[rank] is local
  char* arenaMc;                      // multicast alias of the arena (NULL without NVLS)
  uint32_t* epochs;                   // local device memory: u32 [kMaxBlocks] barrier epochs
  uint32_t* llEpochs;                 // local device memory: u32 [kLLBlocks]
  uint32_t* abortFlag;                // mapped host word; non-zero = give up
  uint32_t* status;                   // mapped host u32 [8]: code, rank, peer, step, block
  uint64_t timeoutNs;                 // budget of one device-side wait
};

// Error codes a kernel can leave in status[0].
enum DevStatus : uint32_t {
  DEV_OK = 0,
  DEV_TIMEOUT_BARRIER = 1,
  DEV_TIMEOUT_LL = 2,
  DEV_TIMEOUT_P2P = 3,
  DEV_TIMEOUT_NET = 4,
  DEV_TIMEOUT_SIGNAL = 5,
  DEV_TIMEOUT_GEMM = 6,
  DEV_TIMEOUT_MOE = 7,
  DEV_ABORTED = 100,
};

}  // namespace uccl
