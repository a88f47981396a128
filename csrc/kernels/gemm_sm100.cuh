// Persistent warp-specialised bf16 GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T (both K-major,
// i.e. the torch.nn.Linear layout), fp32 accumulation in TMEM, optionally fused with the
// tensor-parallel collective next to it.
//
//   warp 0      TMA producer : streams A and B tiles through a shared-memory ring, 128-byte swizzle
//   warp 1      MMA issuer   : one elected lane issues tcgen05.mma, accumulators double-buffered in
//                              TMEM (2 x 256 columns) so the epilogue of tile i overlaps the main
//                              loop of tile i+1
//   warps 2..5  epilogue     : tcgen05.ld TMEM -> registers -> bf16 -> global (or -> shared -> TMA
//                              store into the owning rank's memory, for the reduce-scatter fusion)
//
// Two kernels share this structure: gemm_bf16_kernel (one CTA per 128 x 256 tile) and
// gemm2_bf16_kernel (a cluster of two CTAs per 256 x 256 tile, tcgen05 cta_group::2).
//
// Fusions (the reference has no GEMM at all; these exist for the tensor-parallel MLP block):
//   all-gather -> GEMM : the GEMM producer waits on an arrival counter per 128-row block of A and
//       reads this rank's own rows from the shard itself; tiles are visited in arrival order.  The
//       rows are moved either by copy engines on side streams (host side, see
//       allGatherPushBegin), or by the first `comm_ctas` CTAs of the launch, or by a forwarder
//       warp in every GEMM CTA ("spread"); the last two run comm_allgather_push: bulk TMA copies
//       local shard -> shared memory -> the same rows of every rank's A buffer, and an add to the
//       receiving rank's counter once the copies of a piece have completed.
//   GEMM -> reduce-scatter : the epilogue converts each accumulator tile to bf16, stages it in
//       shared memory and TMA-stores it straight into slot [my rank] of the staging buffer of the
//       rank that owns those rows; the accumulator is handed back to the MMA warp as soon as it
//       has been read, and the owner's counter for the row block is bumped one tile later, when
//       the stores have completed.  When its tiles are done every CTA helps to sum the n staged
//       copies of this rank's own rows in fp32 (local loads only) into the output.  No SM is
//       reserved for communication.
// Every TMA load writes only the shared memory of the CTA that issued it; peers' memory is
// reached with plain (non-replicating) bulk copies.
//
// Every wait is bounded: on expiry the CTA sets a shared bail word, records an error code in
// *args.err, releases TMEM and returns.
#pragma once
#include <cuda.h>
#include "ptx.cuh"

// Phase-skipping switches (Args.debug) and in-kernel time stamps (Args.times) exist only in builds
// made with UCCL_EXPERIMENTS=1 (benchmarks/tp_breakdown.py); product builds compile them out.
#ifdef UCCL_EXPERIMENTS
#define UCCL_DBG(a, bit) (((a).debug & (bit)) != 0)
#define UCCL_TIMES(a) ((a).times)
#else
#define UCCL_DBG(a, bit) false
#define UCCL_TIMES(a) static_cast<unsigned long long*>(nullptr)
#endif

namespace uccl {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int NUM_THREADS_FWD = 224;  // all-gather fusion: one more warp, the forwarder of "spread" mode
constexpr int TMEM_COLS = 512;

// single-CTA kernel: 4 stages of (A 16 KiB + B 32 KiB)
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
// CTA-pair kernel: 6 stages of (A 16 KiB + half of B 16 KiB)
namespace pair {
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = (BN / 2) * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
}  // namespace pair
constexpr int PIPE_BYTES = STAGES * STAGE_BYTES;  // 192 KiB in both kernels
static_assert(PIPE_BYTES == pair::STAGES * pair::STAGE_BYTES, "both kernels share one shared-memory layout");
// epilogue staging for the reduce-scatter fusion: 4 warps x 2 buffers x (32 rows x 128 B)
constexpr int EPI_BUF_BYTES = 32 * 128;
constexpr int EPI_STAGE_BYTES = 4 * 2 * EPI_BUF_BYTES;  // 32 KiB
constexpr int SMEM_BYTES = PIPE_BYTES + EPI_STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

// communication CTAs of the all-gather fusion: six slots of 32 KiB, used in two halves of three
constexpr int COPY_SLOT_BYTES = 32 << 10;
constexpr int COPY_SLOTS = 6;

enum Epilogue : int {
  kEpiStore = 0,   // C[M,N] bf16
  kEpiSwiGLU = 1,  // B rows of a tile are [128 gate rows | 128 up rows]; C[M,N/2] = silu(g)*u
};
enum CommRole : int {
  kCommNone = 0,
  kCommAllGather = 1,
  kCommReduceScatter = 2,    // epilogue TMA-stores tiles into the owners' staging slots
};

constexpr int kMaxPeers = 16;
// Cross-rank flags and counters are one per 128-byte line: hundreds of waiting CTAs poll them,
// and polls of neighbouring words would all land on one L2 line.
constexpr int FLAG_STRIDE = 32;  // in 32-bit words

struct CommArgs {
  int rank = 0;
  int nranks = 1;
  uint64_t timeout_ns = 0;         // deadline for cross-rank waits
  uint32_t* abort_flag = nullptr;  // comm-wide abort word (device-visible)
  // rank barrier folded into the launch: GEMM CTA 0 meets CTA 0 of every rank, then raises `go`;
  // nothing is written to a peer before that
  uint32_t* bar_row_peer[kMaxPeers] = {};  // every rank's barrier words of the fused kernels' slot, indexed by source rank
  uint32_t* bar_epoch = nullptr;            // local: barriers done so far on that slot
  uint32_t* go = nullptr;                   // local, zero at launch: 1 = every rank has arrived, 2 = gave up; nullptr = no folded barrier
  int rows_per_rank = 0;           // multiple of 128
  // all-gather: A_full is a symmetric [M, K] buffer; my shard is pushed into rows
  // [rank * rows_per_rank, ...) of every rank's copy (my own included unless it is already there)
  const char* a_shard = nullptr;
  int a_inplace = 0;
  char* a_full_peer[kMaxPeers] = {};
  uint32_t* ready_peer[kMaxPeers] = {};  // every rank's arrival counters, one per 128-row block, zero at launch
  // reduce-scatter: every rank owns a staging buffer [nranks][rows_per_rank][N]; slot s receives
  // rank s's partial result for the owner's rows (tensor maps in PeerMaps)
  const char* stage_local = nullptr;
  uint32_t* done_peer[kMaxPeers] = {};  // every rank's per-row-block counters, zero at launch
  uint32_t done_target = 0;             // nranks * column tiles
  char* rs_out = nullptr;               // [rows_per_rank, N] bf16
  uint32_t* tail_next = nullptr;        // local, zero at launch: next unit of the summing tail to hand out (nullptr: static split)
  int rs_ldo = 0;
};

// Tensor maps of every rank's reduce-scatter staging buffer ([nranks * rows_per_rank, N] bf16,
// 64-column x 32-row boxes, 128-byte swizzle).
struct PeerMaps {
  CUtensorMap m[kMaxPeers + 1];
};

struct Args {
  int M, N, K;
  __nv_bfloat16* C;
  int ldc;
  int tiles_m, tiles_n;
  int gemm_ctas;            // number of CTAs that run the GEMM roles
  int comm_ctas;            // CTAs [0, comm_ctas) run the communication role (scheduled first)
  int m_rot;                // row-block rotation: logical block i maps to (i + m_rot) % tiles_m
  int m_order;              // 0: rotation only; 1: all-gather order; 2: reduce-scatter order;
                            // 3: all-gather, one peer after the other; 4: reduce-scatter, slab by slab
  int m_bpr;                // 128-row blocks per rank shard (fused modes)
  int b_half_rows;          // SwiGLU: row offset of the "up" half inside B; plain: unused
  const uint32_t* a_ready;  // optional arrival flags per 128-row block (local memory)
  uint32_t a_ready_target;
  int a_local_lo, a_local_hi;  // row blocks in [lo, hi) need no wait (my own rows)
  int a_spread;             // all-gather: warp 6 of every GEMM CTA forwards a share of the shard
  int a_own_shard;          // all-gather: read my own rows through pm.m[0] (the shard) instead of A
  int epi_tma;              // epilogue writes C through shared memory + TMA stores (pm.m[kMaxPeers] maps C)
  uint32_t* err;            // error word (mapped or device memory); 0 = ok
  unsigned long long* times;  // optional: CTA 0 records globaltimer stamps here (profiling aid)
  int debug;                // experiment switches: 1 no communication work, 2 no remote tile stores,
                            // 4 natural tile order, 8 no flag waits, 16 reduce-scatter tiles stay local,
                            // 32 / 64 all-gather without remote / local copies
  CommArgs comm;
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// Bounded wait until *flag >= target. Returns false on timeout / abort.
// Relaxed polls with a growing pause, one system-scope fence on success.
__device__ __forceinline__ bool wait_flag_geq(const uint32_t* flag, uint32_t target, uint64_t timeout_ns,
                                              const uint32_t* abort_flag) {
  if (ptx::ld_relaxed_sys_u32(flag) >= target) {
    ptx::fence_sys();
    return true;
  }
  const uint64_t t0 = ptx::globaltimer_ns();
  const uint64_t limit = timeout_ns ? timeout_ns : 10000000000ull;  // never without a deadline
  uint32_t spins = 0, pause = 32;
  while (true) {
    if (ptx::ld_relaxed_sys_u32(flag) >= target) {
      ptx::fence_sys();
      return true;
    }
    if ((++spins & 63u) == 0) {
      if (abort_flag && ptx::ld_relaxed_sys_u32(abort_flag)) return false;
      if (ptx::globaltimer_ns() - t0 > limit) return false;
    }
    __nanosleep(pause);
    if (pause < 1024) pause <<= 1;
  }
}

// The launch's rank barrier, run by lanes 1 .. nranks of one otherwise idle warp of GEMM CTA 0
// (lane p + 1 deals with rank p) while the GEMM roles already work on tiles that need no peer:
// same words and epochs as the collectives' CTA barrier (coll_device.cuh rank_barrier), on a slot
// of its own.  Raises `go` for everybody who is about to touch a peer.
__device__ __forceinline__ void prologue_barrier(const CommArgs& c, int lane, uint32_t* err) {
  if (lane < 1 || lane > c.nranks) return;
  const unsigned mask = ((c.nranks >= 31 ? 0xffffffffu : ((1u << (c.nranks + 1)) - 1u))) & ~1u;
  const int p = lane - 1;
  const uint32_t e = *c.bar_epoch + 1;
  ptx::fence_sys();
  ptx::st_release_sys_u32(c.bar_row_peer[p] + c.rank, e);
  const uint32_t* mine = c.bar_row_peer[c.rank] + p;
  bool ok = true;
  const uint64_t t0 = ptx::globaltimer_ns();
  const uint64_t limit = c.timeout_ns ? c.timeout_ns : 10000000000ull;
  uint32_t spins = 0;
  while (static_cast<int32_t>(ptx::ld_relaxed_sys_u32(mine) - e) < 0) {
    if ((++spins & 31u) == 0) {
      if ((c.abort_flag && ptx::ld_relaxed_sys_u32(c.abort_flag)) || ptx::globaltimer_ns() - t0 > limit) {
        ok = false;
        break;
      }
    }
  }
  ptx::fence_sys();
  const bool all = __all_sync(mask, ok);
  if (lane == 1) {
    *c.bar_epoch = e;  // advance even on failure: the peers did too
    if (!all && err) atomicCAS(err, 0u, 0x42415252u);
    __threadfence();
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(c.go), "r"(all ? 1u : 2u) : "memory");
  }
}
// Wait for the folded barrier (one thread).  True when every rank has arrived.
__device__ __forceinline__ bool wait_go(const CommArgs& c) {
  if (!c.go) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  const uint64_t limit = (c.timeout_ns ? c.timeout_ns : 10000000000ull) + 1000000000ull;
  uint32_t spins = 0, v;
  while (true) {
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(c.go) : "memory");
    if (v != 0) return v == 1;
    if ((++spins & 63u) == 0 && ptx::globaltimer_ns() - t0 > limit) return false;
    __nanosleep(64);
  }
}

// logical row-block index (in units of `unit` 128-row blocks per tile row) -> physical
__device__ __forceinline__ int order_rows(const Args& a, int m, int tiles_rows, int unit) {
  if (a.m_order == 1) {
    // all-gather: my own shard first (it is already here), then row block j of every other
    // shard for j = 0, 1, ... -- the order in which the pushed blocks arrive
    const int bpr = a.m_bpr / unit, n = a.comm.nranks, r = a.comm.rank;
    if (m < bpr) return r * bpr + m;
    const int i = m - bpr, j = i / (n - 1), q = i % (n - 1) + 1;
    return ((r + q) % n) * bpr + j;
  }
  if (a.m_order == 3) {
    // all-gather by copy-engine lanes: my own shard, then the whole shard of rank r+1, r+2, ...
    const int bpr = a.m_bpr / unit, n = a.comm.nranks, r = a.comm.rank;
    if (m < bpr) return r * bpr + m;
    const int i = m - bpr, q = i / bpr + 1, j = i - (q - 1) * bpr;
    return ((r + q) % n) * bpr + j;
  }
  if (a.m_order == 2) {
    // reduce-scatter: row block j of every shard in turn, each rank starting at its own shard,
    // so that the traffic into every owner is spread over the whole run
    const int bpr = a.m_bpr / unit, n = a.comm.nranks;
    const int j = m / n, s = (m % n + a.comm.rank) % n;
    return s * bpr + j;
  }
  m += a.m_rot;
  return m >= tiles_rows ? m - tiles_rows : m;
}

// tile index -> (row tile, column tile): GROUP consecutive row tiles share a column tile sweep
template <int GROUP>
__device__ __forceinline__ void tile_coords(const Args& a, int tile, int tiles_rows, int unit, int& mrow, int& nb) {
  const int per_group = GROUP * a.tiles_n;
  const int g = tile / per_group;
  const int first = g * GROUP;
  const int gsz = min(GROUP, tiles_rows - first);
  const int r = tile - g * per_group;
  nb = r / gsz;
  mrow = order_rows(a, first + (r % gsz), tiles_rows, unit);
}

// ------------------------------------------------------------------ all-gather push
// The shard is cut into pieces of SLOT_BYTES, dealt round-robin to the participating CTAs.  One
// thread per CTA runs a ring of SLOTS shared-memory slots: local bulk load of piece k+AHEAD, bulk
// stores of piece k to every other rank, and - LAG pieces later, when those stores have completed -
// the arrival counters of the piece's row block on every rank.
// Two users: dedicated communication CTAs (six 32 KiB slots in the pipeline's shared memory), and
// the forwarder warp that every GEMM CTA has in "spread" mode (four 8 KiB slots in the epilogue
// staging area, which the all-gather fusion does not use).  A single SM sustains only about
// 20 GB/s of remote stores, so the second form, which spreads the shard over all SMs and takes
// none of them away from the GEMM, is the one that can fill the links.
constexpr int FWD_SLOT_BYTES = 8 << 10;
constexpr int FWD_SLOTS = 4;

template <int SLOT_BYTES, int SLOTS, int AHEAD, int LAG>
__device__ void comm_allgather_push(const Args& a, uint8_t* smem, uint64_t* bars, int cta, int nctas) {
  static_assert(AHEAD < SLOTS, "some slots must be left to the stores");
  const CommArgs& c = a.comm;
  const int n = c.nranks, r = c.rank, bpr = a.m_bpr;
  const size_t blkBytes = static_cast<size_t>(BM) * a.K * 2;
  const int nsub = static_cast<int>((blkBytes + SLOT_BYTES - 1) / SLOT_BYTES);
  const int allPieces = bpr * nsub;
  const size_t shardOff = static_cast<size_t>(r) * bpr * blkBytes;
  uint64_t* full = bars;  // SLOTS barriers
  for (int s = 0; s < SLOTS; ++s) ptx::mbar_init(&full[s], 1);
  ptx::mbar_fence_init();
  volatile uint32_t bail = 0;
#ifdef UCCL_EXPERIMENTS
  const int mapMode = (a.debug >> 10) & 3;  // experiments: 1 whole blocks per CTA, 2 one contiguous range per CTA
#else
  constexpr int mapMode = 0;
#endif
  int total = 0;
  if (mapMode == 0) {
    for (int g = cta; g < allPieces; g += nctas) ++total;
  } else if (mapMode == 1) {
    for (int b = cta; b < bpr; b += nctas) total += nsub;
  } else {
    const int per = (allPieces + nctas - 1) / nctas;
    total = max(0, min(per, allPieces - cta * per));
  }
  auto piece = [&](int i) {
    if (mapMode == 0) return cta + i * nctas;
    if (mapMode == 1) return (cta + (i / nsub) * nctas) * nsub + i % nsub;
    return cta * ((allPieces + nctas - 1) / nctas) + i;
  };
  auto where = [&](int i, size_t& off, uint32_t& bytes, int& blk) {
    const int g = piece(i);
    blk = g / nsub;
    const int sub = g - blk * nsub;
    off = static_cast<size_t>(blk) * blkBytes + static_cast<size_t>(sub) * SLOT_BYTES;
    const size_t left = blkBytes - static_cast<size_t>(sub) * SLOT_BYTES;
    bytes = static_cast<uint32_t>(left < SLOT_BYTES ? left : SLOT_BYTES);
  };
  // arrival counters: one add per (row block, rank) covering this CTA's pieces of the block
  int curBlk = -1;
  uint32_t cnt = 0;
  auto flush = [&]() {
    if (curBlk < 0 || cnt == 0) return;
    // the counted stores have completed (wait_group), which makes them visible to this thread;
    // the fence orders them before the counter updates.  No proxy fence here: it would also wait
    // for the newer stores that are still in flight.
    ptx::fence_sys();
    for (int q = 1; q < n; ++q) {
      const int p = (r + q) % n;
      ptx::red_relaxed_sys_add_u32(c.ready_peer[p] + static_cast<size_t>(r * bpr + curBlk) * FLAG_STRIDE, cnt);
    }
    cnt = 0;
  };
  auto completed = [&](int i) {
    size_t off; uint32_t bytes; int blk;
    where(i, off, bytes, blk);
    if (blk != curBlk) {
      flush();
      curBlk = blk;
    }
    ++cnt;
    if (i + 1 >= total || piece(i + 1) / nsub != blk) flush();
  };
  auto load = [&](int i) {
    size_t off; uint32_t bytes; int blk;
    where(i, off, bytes, blk);
    const int slot = i % SLOTS;
    ptx::mbar_expect_tx(&full[slot], bytes);
    ptx::bulk_load(smem + slot * SLOT_BYTES, c.a_shard + off, bytes, &full[slot]);
  };
  for (int i = 0; i < AHEAD && i < total; ++i) load(i);
  for (int k = 0; k < total; ++k) {
    size_t off; uint32_t bytes; int blk;
    where(k, off, bytes, blk);
    const int slot = k % SLOTS;
    if (!ptx::mbar_wait_bounded(&full[slot], (k / SLOTS) & 1, &bail)) {
      if (a.err) atomicCAS(a.err, 0u, 0x41475000u | static_cast<uint32_t>(blk & 0xfff));
      ptx::tma_store_wait<0>();
      return;
    }
    for (int q = 1; q < n; ++q) {
      const int p = (r + 1 + (q - 1 + k) % (n - 1)) % n;  // start at a different rank for every piece
      ptx::bulk_store(c.a_full_peer[p] + shardOff + off, smem + slot * SLOT_BYTES, bytes);
    }
    ptx::tma_store_commit();
    ptx::tma_store_wait_read<SLOTS - AHEAD>();  // pieces <= k-2 have left shared memory
    if (k + AHEAD < total) load(k + AHEAD);
    if (k >= LAG) {
      ptx::tma_store_wait<LAG>();  // the stores of pieces <= k-LAG have completed on every rank
      completed(k - LAG);
    }
  }
  ptx::tma_store_wait<0>();
  for (int i = total > LAG ? total - LAG : 0; i < total; ++i) completed(i);
  flush();
}

// ------------------------------------------------------------------ reduce-scatter tail (all GEMM CTAs)
// out[row, :] = sum over source ranks of stage[src][row, :] for this rank's rows, fp32 accumulate.
// Every thread keeps sixteen 16-byte loads in flight (V vectors x n sources).
template <int V>
__device__ __forceinline__ void tail_rows(const CommArgs& c, int n, size_t slotBytes, size_t rowBytes, int vecPerRow,
                                          size_t row0, int nvec) {
  // vector v of a thread is blockDim.x vectors after its vector v-1: every load is coalesced
  const int T = blockDim.x;
  for (int i0 = threadIdx.x; i0 < nvec; i0 += T * V) {
    float acc[V][8];
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[v][e] = 0.f;
    size_t off[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int i = min(i0 + v * T, nvec - 1);
      const int rr = i / vecPerRow, cv = i - rr * vecPerRow;
      off[v] = (row0 + rr) * rowBytes + (static_cast<size_t>(cv) << 4);
    }
    constexpr int P = 16 / V;  // sources per round
    for (int p0 = 0; p0 < n; p0 += P) {
      uint4 d[V][P];
#pragma unroll
      for (int j = 0; j < P; ++j)
#pragma unroll
        for (int v = 0; v < V; ++v)
          if (p0 + j < n) d[v][j] = ptx::ld_stream_v4(c.stage_local + static_cast<size_t>(p0 + j) * slotBytes + off[v]);
#pragma unroll
      for (int j = 0; j < P; ++j)
#pragma unroll
        for (int v = 0; v < V; ++v)
          if (p0 + j < n) {
            const uint32_t w[4] = {d[v][j].x, d[v][j].y, d[v][j].z, d[v][j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = ptx::unpack_bf16x2(w[e]);
              acc[v][2 * e] += f.x;
              acc[v][2 * e + 1] += f.y;
            }
          }
    }
#pragma unroll
    for (int v = 0; v < V; ++v) {
      if (i0 + v * T < nvec) {
        const int i = i0 + v * T;
        const int rr = i / vecPerRow, cv = i - rr * vecPerRow;
        uint4 o;
        o.x = ptx::pack_bf16x2(acc[v][0], acc[v][1]);
        o.y = ptx::pack_bf16x2(acc[v][2], acc[v][3]);
        o.z = ptx::pack_bf16x2(acc[v][4], acc[v][5]);
        o.w = ptx::pack_bf16x2(acc[v][6], acc[v][7]);
        ptx::st_global_v4(c.rs_out + (row0 + rr) * static_cast<size_t>(c.rs_ldo) * 2 + (static_cast<size_t>(cv) << 4), o);
      }
    }
  }
}

// Register path: used when the shape does not fit the shared-memory ring below.
__device__ void reduce_scatter_tail_direct(const Args& a, int cta, int nctas) {
  const CommArgs& c = a.comm;
  const int n = c.nranks, bpr = a.m_bpr;
  constexpr int SPLIT = 16;              // units per 128-row block: 8 rows each
  constexpr int ROWS = BM / SPLIT;
  const size_t rowBytes = static_cast<size_t>(a.N) * 2;
  const size_t slotBytes = static_cast<size_t>(c.rows_per_rank) * rowBytes;
  const int vecPerRow = static_cast<int>(rowBytes >> 4);
  __shared__ int s_ok;
  const int first_blk = c.rank * bpr;
  for (int u = cta; u < bpr * SPLIT; u += nctas) {
    const int b = u / SPLIT, part = u % SPLIT;
    __syncthreads();
    if (threadIdx.x == 0) {
      const bool ok = wait_flag_geq(c.done_peer[c.rank] + static_cast<size_t>(first_blk + b) * FLAG_STRIDE, c.done_target,
                                    c.timeout_ns, c.abort_flag);
      if (!ok && a.err) atomicCAS(a.err, 0u, 0x52530000u | static_cast<uint32_t>(b));
      s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!s_ok) return;
    const size_t row0 = static_cast<size_t>(b) * BM + part * ROWS;
    const int nvec = ROWS * vecPerRow;
    if (n <= 2) tail_rows<8>(c, n, slotBytes, rowBytes, vecPerRow, row0, nvec);
    else if (n <= 4) tail_rows<4>(c, n, slotBytes, rowBytes, vecPerRow, row0, nvec);
    else tail_rows<2>(c, n, slotBytes, rowBytes, vecPerRow, row0, nvec);
  }
}

// Sum of NR staged copies (NR = 0: n is only known at run time) of one piece held in shared
// memory, written out as bf16.  `dst` is the output address of the piece's first byte when the
// output rows are contiguous; otherwise rows are resolved with 32-bit arithmetic.
template <int NR>
__device__ __forceinline__ void tail_sum_piece(const uint8_t* sbase, uint32_t P, int n, int nv, char* dst, bool contig,
                                               char* out, uint32_t row0, uint32_t colb0, uint32_t rowBytes,
                                               size_t outRowBytes, int t, int nt) {
  // V vectors per step with all their shared-memory loads issued first (about eight in flight)
  constexpr int V = NR == 0 ? 1 : (NR <= 2 ? 4 : (NR <= 4 ? 2 : 1));
  constexpr int NL = NR == 0 ? 1 : NR;
  const int nn = NR > 0 ? NR : n;
  for (int v0 = t; v0 < nv; v0 += V * nt) {
    float acc[V][8];
#pragma unroll
    for (int j = 0; j < V; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
    for (int p0 = 0; p0 < nn; p0 += NL) {
      uint4 d[V][NL];
#pragma unroll
      for (int j = 0; j < V; ++j)
#pragma unroll
        for (int p = 0; p < NL; ++p) {
          const int v = min(v0 + j * nt, nv - 1);
          d[j][p] = *reinterpret_cast<const uint4*>(sbase + static_cast<uint32_t>(p0 + p) * P + (static_cast<uint32_t>(v) << 4));
        }
#pragma unroll
      for (int j = 0; j < V; ++j)
#pragma unroll
        for (int p = 0; p < NL; ++p) {
          const uint32_t w[4] = {d[j][p].x, d[j][p].y, d[j][p].z, d[j][p].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = ptx::unpack_bf16x2(w[e]);
            acc[j][2 * e] += f.x;
            acc[j][2 * e + 1] += f.y;
          }
        }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const int v = v0 + j * nt;
      if (v < nv) {
        uint4 o;
        o.x = ptx::pack_bf16x2(acc[j][0], acc[j][1]);
        o.y = ptx::pack_bf16x2(acc[j][2], acc[j][3]);
        o.z = ptx::pack_bf16x2(acc[j][4], acc[j][5]);
        o.w = ptx::pack_bf16x2(acc[j][6], acc[j][7]);
        char* q;
        if (contig) {
          q = dst + (static_cast<uint32_t>(v) << 4);
        } else {
          const uint32_t tb = colb0 + (static_cast<uint32_t>(v) << 4);
          const uint32_t dr = tb / rowBytes;
          q = out + static_cast<size_t>(row0 + dr) * outRowBytes + (tb - dr * rowBytes);
        }
        *reinterpret_cast<uint4*>(q) = o;  // the output is private to this rank: a plain store
      }
    }
  }
}

// Main path: the pipeline's shared memory (idle once the CTA's tiles are done) becomes a ring of
// three 64 KiB stages.  Warp 0 is the loader: one thread checks the row block's counter and
// bulk-loads the n staged copies of one piece of the block into a stage; warps 1-5 add them up
// from shared memory and write the bf16 result.  192 KiB of loads in flight per SM without
// holding them in registers.
__device__ void reduce_scatter_tail(const Args& a, uint8_t* smem, uint64_t* tbars, volatile uint32_t* bail, int cta,
                                    int nctas) {
  const CommArgs& c = a.comm;
  const int n = c.nranks, bpr = a.m_bpr;
  constexpr int TSTAGES = 3;
  constexpr uint32_t TSTAGE_BYTES = 64u << 10;
  const size_t rowBytes = static_cast<size_t>(a.N) * 2;
  const size_t blkBytes = static_cast<size_t>(BM) * rowBytes;
  const size_t slotBytes = static_cast<size_t>(c.rows_per_rank) * rowBytes;
  // pieces per row block: a power of two with n * piece <= stage size, piece a multiple of 16 bytes
  int pieces = 1;
  while (pieces < 4096 && (blkBytes / pieces) * n > TSTAGE_BYTES) pieces <<= 1;
  if ((blkBytes % pieces) != 0 || ((blkBytes / pieces) & 15) != 0 || (blkBytes / pieces) * n > TSTAGE_BYTES ||
      rowBytes > 0x7fffffffu) {
    reduce_scatter_tail_direct(a, cta, nctas);
    return;
  }
  const uint32_t P = static_cast<uint32_t>(blkBytes / pieces);
  const int units = bpr * pieces;
  // Units (one piece of one row block) are handed out in block order, which is the order in which
  // the blocks complete: from a shared counter when the launch has one, so that reducer CTAs that
  // start at once and GEMM CTAs that join when their tiles are done share the work; else by a
  // static stride over the CTAs.
  __shared__ int s_unit[3];
  int claimed = 0;  // thread 0: claims made so far (static split)
  auto claim = [&]() -> int {
    int u;
    if (c.tail_next) u = static_cast<int>(atomicAdd(c.tail_next, 1u));
    else u = cta + (claimed++) * nctas;
    return u < units ? u : -1;
  };
  const int first_blk = c.rank * bpr;
  uint32_t* done = c.done_peer[c.rank] + static_cast<size_t>(first_blk) * FLAG_STRIDE;
  // blocks [0, readyUpTo) are known complete; counters are read relaxed and one fence follows
  int readyUpTo = 0;
  if (threadIdx.x == 0) {
    for (int i = 0; i < TSTAGES; ++i) ptx::mbar_init(&tbars[i], 1);
    ptx::mbar_fence_init();
  }
  // Row block b of mine is complete when its counter has every rank's tiles.
  auto peek = [&](int b) -> bool {
    return ptx::ld_relaxed_sys_u32(done + static_cast<size_t>(b) * FLAG_STRIDE) >= c.done_target;
  };
  auto await = [&](int b) -> bool {  // bounded; thread 0 only
    return wait_flag_geq(done + static_cast<size_t>(b) * FLAG_STRIDE, c.done_target, c.timeout_ns, c.abort_flag);
  };
  // every thread looks at one row block; the loader takes the complete prefix
  uint32_t* s_ready = reinterpret_cast<uint32_t*>(smem);  // [bpr] flags, shared memory is idle here
  for (int b = threadIdx.x; b < bpr; b += blockDim.x) s_ready[b] = peek(b) ? 1u : 0u;
  __syncthreads();
  if (threadIdx.x == 0) {
    while (readyUpTo < bpr && s_ready[readyUpTo]) ++readyUpTo;
    ptx::fence_sys();
    ptx::fence_proxy_async();  // the staged tiles were written by the ranks' TMA stores
  }
  __syncthreads();
  auto issue = [&](int i) {  // thread 0: claims my i-th unit and starts its loads
    const int u = claim();
    s_unit[i % TSTAGES] = u;
    if (u < 0) return;
    const int b = u / pieces, part = u - b * pieces;
    if (b >= readyUpTo) {
      if (!await(b)) {
        if (a.err) atomicCAS(a.err, 0u, 0x52530000u | static_cast<uint32_t>(b));
        *bail = 1;
        return;
      }
      ptx::fence_proxy_async();
      if (b == readyUpTo) ++readyUpTo;
    }
    const int st = i % TSTAGES;
    ptx::mbar_expect_tx(&tbars[st], static_cast<uint32_t>(n) * P);
    const size_t off = static_cast<size_t>(b) * blkBytes + static_cast<size_t>(part) * P;
    for (int p = 0; p < n; ++p)
      ptx::bulk_load(smem + st * TSTAGE_BYTES + static_cast<uint32_t>(p) * P,
                     c.stage_local + static_cast<size_t>(p) * slotBytes + off, P, &tbars[st]);
  };
  if (threadIdx.x == 0) {
    for (int i = 0; i < TSTAGES - 1; ++i) {
      if (!*bail) issue(i);
      else s_unit[i] = -1;
    }
  }
  __syncthreads();
  const int nv = static_cast<int>(P >> 4);
  const bool contig = static_cast<size_t>(c.rs_ldo) * 2 == rowBytes;
  const size_t outRowBytes = static_cast<size_t>(c.rs_ldo) * 2;
  const int warp = threadIdx.x >> 5;
  if (UCCL_TIMES(a) && cta == 0 && threadIdx.x == 0) a.times[2] = ptx::globaltimer_ns();
  for (int i = 0;; ++i) {
    // stage (i + 2) % 3 was consumed in iteration i - 1, which ended with a CTA barrier
    if (threadIdx.x == 0) {
      if (!*bail) issue(i + TSTAGES - 1);
      else s_unit[(i + TSTAGES - 1) % TSTAGES] = -1;
    }
    const int st = i % TSTAGES;
    const int u = s_unit[st];  // written two iterations (two CTA barriers) ago
    if (u < 0) break;  // same value in every thread
    bool ok = true;
    if (warp != 0) ok = ptx::mbar_wait_bounded(&tbars[st], (i / TSTAGES) & 1, bail);
    if (UCCL_TIMES(a) && cta == 0 && threadIdx.x == 32 && i < 8) a.times[16 + 2 * i] = ptx::globaltimer_ns();
    if (warp != 0 && ok) {
      const int b = u / pieces, part = u - b * pieces;
      const size_t flat0 = static_cast<size_t>(b) * blkBytes + static_cast<size_t>(part) * P;
      const uint32_t row0 = static_cast<uint32_t>(flat0 / rowBytes);
      const uint32_t colb0 = static_cast<uint32_t>(flat0 - static_cast<size_t>(row0) * rowBytes);
      const uint8_t* sbase = smem + st * TSTAGE_BYTES;
      char* dst = c.rs_out + flat0;
      const int t = threadIdx.x - 32, nt = blockDim.x - 32;
      const uint32_t rb = static_cast<uint32_t>(rowBytes);
      if (n == 2) tail_sum_piece<2>(sbase, P, n, nv, dst, contig, c.rs_out, row0, colb0, rb, outRowBytes, t, nt);
      else if (n == 4) tail_sum_piece<4>(sbase, P, n, nv, dst, contig, c.rs_out, row0, colb0, rb, outRowBytes, t, nt);
      else if (n == 8) tail_sum_piece<8>(sbase, P, n, nv, dst, contig, c.rs_out, row0, colb0, rb, outRowBytes, t, nt);
      else tail_sum_piece<0>(sbase, P, n, nv, dst, contig, c.rs_out, row0, colb0, rb, outRowBytes, t, nt);
      if (UCCL_TIMES(a) && cta == 0 && threadIdx.x == 32 && i < 8) a.times[17 + 2 * i] = ptx::globaltimer_ns();
    }
    if (__syncthreads_or(ok ? 0 : 1)) break;
    if (UCCL_TIMES(a) && cta == 0 && threadIdx.x == 0 && i < 12) a.times[3 + i] = ptx::globaltimer_ns();
  }
}

// ------------------------------------------------------------------ epilogue of one tile, one warp
// `taddr` addresses this warp's 32 TMEM lanes of the accumulator; `mb` is the 128-row block.
// 64 columns x 32 rows of bf16 (eight 16-byte pieces per lane) -> 128-byte-swizzled staging buffer
// -> one TMA store at (col0, row0) of `map`.  One bulk group per call.
template <int NBUF>
__device__ __forceinline__ void stage_and_store(const CUtensorMap* map, const uint4 (&v)[8], int col0, int row0, bool inside,
                                                int lane, uint8_t* stage, uint32_t& stage_it) {
  uint8_t* buf = stage + (stage_it % NBUF) * EPI_BUF_BYTES;
  ++stage_it;
  if (lane == 0) ptx::tma_store_wait_read<NBUF - 1>();  // the store that last used this buffer has read it
  __syncwarp();
  uint8_t* myrow = buf + lane * 128;
#pragma unroll
  for (int k = 0; k < 8; ++k) *reinterpret_cast<uint4*>(myrow + ((k ^ (lane & 7)) << 4)) = v[k];  // 128-byte swizzle
  ptx::fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0 && inside) ptx::tma_store_2d(map, buf, col0, row0);
  if (lane == 0) ptx::tma_store_commit();
}

// `cmap` != nullptr: C is written through shared memory and TMA stores (whole 128-byte lines, rows
// and columns beyond the matrix clipped by the copy engine) at rows crow0 ... of that map; else
// every lane stores its own row with 16-byte stores.
template <int EPI, int COMM, int NBUF>
__device__ __forceinline__ void epilogue_tile(const Args& a, const PeerMaps& pm, uint32_t taddr, int mb, int nb, int q,
                                              int lane, uint8_t* stage, uint32_t& stage_it, __nv_bfloat16* cbase,
                                              const CUtensorMap* cmap = nullptr, int crow0 = 0) {
  const int row = mb * BM + q * 32 + lane;
  if (COMM != kCommReduceScatter && cmap) {
    if (EPI == kEpiStore) {
#pragma unroll 1
      for (int g = 0; g < BN / 64; ++g) {
        uint32_t r0[32], r1[32];
        ptx::tmem_ld_32x32b_x32(taddr + g * 64, r0);
        ptx::tmem_ld_32x32b_x32(taddr + g * 64 + 32, r1);
        ptx::tmem_ld_wait();
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t* s = k < 4 ? &r0[8 * k] : &r1[8 * (k - 4)];
          v[k].x = ptx::pack_bf16x2(__uint_as_float(s[0]), __uint_as_float(s[1]));
          v[k].y = ptx::pack_bf16x2(__uint_as_float(s[2]), __uint_as_float(s[3]));
          v[k].z = ptx::pack_bf16x2(__uint_as_float(s[4]), __uint_as_float(s[5]));
          v[k].w = ptx::pack_bf16x2(__uint_as_float(s[6]), __uint_as_float(s[7]));
        }
        const int col0 = nb * BN + g * 64;
        stage_and_store<NBUF>(cmap, v, col0, crow0, col0 < a.N && crow0 < a.M, lane, stage, stage_it);
      }
    } else {
      // gate columns [0,128) and up columns [128,256) of the accumulator -> 128 output columns
      const int out_n = a.N / 2;
#pragma unroll 1
      for (int g = 0; g < BN / 128; ++g) {
        uint4 v[8];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t gt[32], up[32];
          ptx::tmem_ld_32x32b_x32(taddr + g * 64 + h * 32, gt);
          ptx::tmem_ld_32x32b_x32(taddr + BN / 2 + g * 64 + h * 32, up);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = silu_f(__uint_as_float(gt[8 * j + e])) * __uint_as_float(up[8 * j + e]);
            v[h * 4 + j].x = ptx::pack_bf16x2(o[0], o[1]);
            v[h * 4 + j].y = ptx::pack_bf16x2(o[2], o[3]);
            v[h * 4 + j].z = ptx::pack_bf16x2(o[4], o[5]);
            v[h * 4 + j].w = ptx::pack_bf16x2(o[6], o[7]);
          }
        }
        const int col0 = nb * (BN / 2) + g * 64;
        stage_and_store<NBUF>(cmap, v, col0, crow0, col0 < out_n && crow0 < a.M, lane, stage, stage_it);
      }
    }
    return;
  }
  if (COMM == kCommReduceScatter) {
    // bf16 tile -> swizzled shared memory -> TMA store into the owner's staging slot [my rank]
    const int rpr = a.comm.rows_per_rank;
    const int owner = min((mb * BM) / rpr, a.comm.nranks - 1);
    const int drow = a.comm.rank * rpr + (mb * BM + q * 32 - owner * rpr);
    const CUtensorMap* dmap = &pm.m[UCCL_DBG(a, 16) ? a.comm.rank : owner];
#pragma unroll 1
    for (int g = 0; g < BN / 64; ++g) {
      uint32_t r0[32], r1[32];
      ptx::tmem_ld_32x32b_x32(taddr + g * 64, r0);
      ptx::tmem_ld_32x32b_x32(taddr + g * 64 + 32, r1);
      ptx::tmem_ld_wait();
      uint8_t* buf = stage + (stage_it % NBUF) * EPI_BUF_BYTES;
      ++stage_it;
      if (lane == 0) ptx::tma_store_wait_read<NBUF - 1>();  // the store that last used this buffer has read it
      __syncwarp();
      uint8_t* myrow = buf + lane * 128;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t* s = k < 4 ? &r0[8 * k] : &r1[8 * (k - 4)];
        uint4 v;
        v.x = ptx::pack_bf16x2(__uint_as_float(s[0]), __uint_as_float(s[1]));
        v.y = ptx::pack_bf16x2(__uint_as_float(s[2]), __uint_as_float(s[3]));
        v.z = ptx::pack_bf16x2(__uint_as_float(s[4]), __uint_as_float(s[5]));
        v.w = ptx::pack_bf16x2(__uint_as_float(s[6]), __uint_as_float(s[7]));
        *reinterpret_cast<uint4*>(myrow + ((k ^ (lane & 7)) << 4)) = v;  // 128-byte swizzle
      }
      const int col0 = nb * BN + g * 64;
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && col0 < a.N && !UCCL_DBG(a, 2)) {
        ptx::tma_store_2d(dmap, buf, col0, drow);
      }
      if (lane == 0) ptx::tma_store_commit();  // exactly BN / 64 groups per tile
    }
    return;  // the caller publishes the tile once these groups have completed
  }
  if (EPI == kEpiStore) {
    __nv_bfloat16* crow = cbase + static_cast<size_t>(row) * a.ldc + static_cast<size_t>(nb) * BN;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
      ptx::tmem_ld_wait();
      const int col0 = nb * BN + c * 32;
      if (row < a.M) {
        if (col0 + 32 <= a.N) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = ptx::pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            v.y = ptx::pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            v.z = ptx::pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            v.w = ptx::pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            *reinterpret_cast<uint4*>(crow + c * 32 + j * 8) = v;
          }
        } else {
          for (int j = 0; j < 32; ++j)
            if (col0 + j < a.N) crow[c * 32 + j] = __float2bfloat16(__uint_as_float(r[j]));
        }
      }
    }
  } else {
    // gate columns [0,128) and up columns [128,256) of the accumulator
    const int out_n = a.N / 2;
    __nv_bfloat16* crow = cbase + static_cast<size_t>(row) * a.ldc + static_cast<size_t>(nb) * (BN / 2);
#pragma unroll 1
    for (int c = 0; c < BN / 64; ++c) {
      uint32_t g[32], u[32];
      ptx::tmem_ld_32x32b_x32(taddr + c * 32, g);
      ptx::tmem_ld_32x32b_x32(taddr + BN / 2 + c * 32, u);
      ptx::tmem_ld_wait();
      const int col0 = nb * (BN / 2) + c * 32;
      if (row < a.M) {
        if (col0 + 32 <= out_n) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float h[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) h[e] = silu_f(__uint_as_float(g[8 * j + e])) * __uint_as_float(u[8 * j + e]);
            uint4 v;
            v.x = ptx::pack_bf16x2(h[0], h[1]);
            v.y = ptx::pack_bf16x2(h[2], h[3]);
            v.z = ptx::pack_bf16x2(h[4], h[5]);
            v.w = ptx::pack_bf16x2(h[6], h[7]);
            *reinterpret_cast<uint4*>(crow + c * 32 + j * 8) = v;
          }
        } else {
          for (int j = 0; j < 32; ++j)
            if (col0 + j < out_n)
              crow[c * 32 + j] = __float2bfloat16(silu_f(__uint_as_float(g[j])) * __uint_as_float(u[j]));
        }
      }
    }
  }
}

// Reduce-scatter bookkeeping of one epilogue warp: the tile it wrote `lag` tiles ago is complete
// once at most `pending` newer bulk groups are outstanding.  The last of the four epilogue warps
// to report a tile tells the owner that one more tile of its row block has landed.  Counters are
// kept per (tile index mod 4): the warps of a CTA are never more than three tiles apart, because
// the MMA warp needs all four to have drained accumulator t-2 before it can produce tile t.
template <int PENDING>
__device__ __forceinline__ void publish_tile(const Args& a, int mb, int lane, uint32_t* counter) {
  if (lane != 0) return;
  ptx::tma_store_wait<PENDING>();
  __threadfence_block();
  const uint32_t old = atomicAdd(counter, 1u);
  if ((old & 3u) == 3u) {
    ptx::fence_sys();
    const int owner = min((mb * BM) / a.comm.rows_per_rank, a.comm.nranks - 1);
    ptx::red_release_sys_add_u32(a.comm.done_peer[owner] + static_cast<size_t>(mb) * FLAG_STRIDE, 1u);
  }
}

// ------------------------------------------------------------------ single-CTA kernel
template <int EPI, int COMM>
__global__ void __launch_bounds__(COMM == kCommAllGather ? NUM_THREADS_FWD : NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ PeerMaps pm, const Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PIPE_BYTES + EPI_STAGE_BYTES);
  if (COMM == kCommAllGather && static_cast<int>(blockIdx.x) < a.comm_ctas) {
    if (!UCCL_DBG(a, 1) && threadIdx.x == 0 && wait_go(a.comm))
      comm_allgather_push<COPY_SLOT_BYTES, COPY_SLOTS, 4, 4>(a, smem, bars, blockIdx.x, a.comm_ctas);
    return;
  }
  const int cta_id = static_cast<int>(blockIdx.x) - a.comm_ctas;
  if (COMM == kCommReduceScatter && cta_id >= a.gemm_ctas) {
    // reducer CTA: sums the staged copies of this rank's row blocks as they complete, from the start
    volatile uint32_t* rbail = reinterpret_cast<volatile uint32_t*>(bars + 28);
    if (threadIdx.x == 0) *rbail = 0;
    __syncthreads();
    reduce_scatter_tail(a, smem, bars + 24, rbail, cta_id, a.gemm_ctas);
    return;
  }
  uint64_t* full_bar = bars;                     // [STAGES]
  uint64_t* empty_bar = bars + STAGES;           // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;       // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* bail = tmem_holder + 1;
  uint32_t* warps_done = tmem_holder + 2;

  if (UCCL_TIMES(a) && cta_id == 0 && threadIdx.x == 0) a.times[0] = ptx::globaltimer_ns();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = a.tiles_m * a.tiles_n;
  const int num_kb = (a.K + BK - 1) / BK;
  const int gemm_ctas = a.gemm_ctas;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&tfull_bar[i], 1);
      ptx::mbar_init(&tempty_bar[i], 4);  // one arrive per epilogue warp
    }
    *bail = 0;
    warps_done[0] = warps_done[1] = warps_done[2] = warps_done[3] = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB);
    if (COMM == kCommAllGather) ptx::prefetch_tmap(&pm.m[0]);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_holder, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = cta_id; tile < num_tiles && !*bail; tile += gemm_ctas) {
        int mb, nb;
        tile_coords<16>(a, tile, a.tiles_m, 1, mb, nb);
        const bool own = mb >= a.a_local_lo && mb < a.a_local_hi;
        if (a.a_ready && !UCCL_DBG(a, 8) && !own) {
          if (!wait_flag_geq(a.a_ready + static_cast<size_t>(mb) * FLAG_STRIDE, a.a_ready_target, a.comm.timeout_ns,
                             a.comm.abort_flag)) {
            if (a.err) atomicCAS(a.err, 0u, 0x41470000u | static_cast<uint32_t>(mb));
            *bail = 1;
            break;
          }
          ptx::fence_proxy_async();  // the rows were written by bulk stores (async proxy)
        }
        // my own rows are read from the shard itself; pm.m[0] is its tensor map
        const bool fromShard = COMM == kCommAllGather && own && a.a_own_shard;
        const CUtensorMap* ta = fromShard ? &pm.m[0] : &tmA;
        const int m0 = fromShard ? (mb - a.a_local_lo) * BM : mb * BM;
        int brow0, brow1;
        if (EPI == kEpiSwiGLU) {
          brow0 = nb * (BN / 2);
          brow1 = a.b_half_rows + nb * (BN / 2);
        } else {
          brow0 = nb * BN;
          brow1 = nb * BN + BN / 2;
        }
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait_bounded(&empty_bar[s], ph ^ 1, bail)) break;
          uint8_t* sA = smem + s * STAGE_BYTES;
          uint8_t* sB = sA + A_STAGE_BYTES;
          ptx::mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          ptx::tma_load_2d(sA, ta, &full_bar[s], kb * BK, m0);
          ptx::tma_load_2d(sB, &tmB, &full_bar[s], kb * BK, brow0);
          ptx::tma_load_2d(sB + B_STAGE_BYTES / 2, &tmB, &full_bar[s], kb * BK, brow1);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::umma_idesc_f16(1u, BM, BN);
      uint32_t it = 0, tcount = 0;
      for (int tile = cta_id; tile < num_tiles && !*bail; tile += gemm_ctas, ++tcount) {
        const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
        if (!ptx::mbar_wait_bounded(&tempty_bar[acc], acc_ph ^ 1, bail)) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!ptx::mbar_wait_bounded(&full_bar[s], ph, bail)) break;
          ptx::tc_fence_after();
          const uint32_t sA = ptx::smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = ptx::umma_smem_desc_sw128(sA);
          const uint64_t db = ptx::umma_smem_desc_sw128(sA + A_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t koff = static_cast<uint64_t>((k * UMMA_K * 2) >> 4);
            ptx::umma_f16(d_tmem, da + koff, db + koff, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[s]);
        }
        ptx::umma_commit(&tfull_bar[acc]);
      }
    } else if (COMM != kCommNone && a.comm.go && cta_id == 0) {
      prologue_barrier(a.comm, lane, a.err);  // the warp's idle lanes run the launch's rank barrier
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ forwarder (all-gather, spread mode)
    int go_ok = 1;
    if (COMM == kCommAllGather && a.a_spread && lane == 0) go_ok = wait_go(a.comm) ? 1 : 0;
    go_ok = __shfl_sync(0xffffffffu, go_ok, 0);
    if (COMM == kCommAllGather && a.a_spread && !UCCL_DBG(a, 1) && go_ok) {
      if (lane == 0) comm_allgather_push<FWD_SLOT_BYTES, FWD_SLOTS, 2, 2>(a, smem + PIPE_BYTES, bars + 24, blockIdx.x, gridDim.x);
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint8_t* stage = smem + PIPE_BYTES + q * 2 * EPI_BUF_BYTES;
    uint32_t tcount = 0, stage_it = 0;
    int prev_mb = 0;
    if (COMM == kCommReduceScatter) {
      // no tile leaves for a peer before every rank has entered this launch
      int g = 1;
      if (lane == 0) g = wait_go(a.comm) ? 1 : 0;
      if (!__shfl_sync(0xffffffffu, g, 0) && lane == 0) *bail = 1;
      __syncwarp();
    }
    for (int tile = cta_id; tile < num_tiles && !*bail; tile += gemm_ctas, ++tcount) {
      int mb, nb;
      tile_coords<16>(a, tile, a.tiles_m, 1, mb, nb);
      const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
      if (!ptx::mbar_wait_bounded(&tfull_bar[acc], acc_ph, bail)) break;
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      epilogue_tile<EPI, COMM, 2>(a, pm, taddr, mb, nb, q, lane, stage, stage_it, a.C,
                                  a.epi_tma ? &pm.m[kMaxPeers] : nullptr, mb * BM + q * 32);
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&tempty_bar[acc]);
      if (COMM == kCommReduceScatter) {
        // the previous tile's stores have had a whole tile to complete
        if (tcount > 0) publish_tile<BN / 64>(a, prev_mb, lane, &warps_done[(tcount - 1) & 3]);
        prev_mb = mb;
      }
    }
    if (COMM == kCommReduceScatter && tcount > 0) publish_tile<0>(a, prev_mb, lane, &warps_done[(tcount - 1) & 3]);
    if (COMM != kCommReduceScatter && a.epi_tma && lane == 0) ptx::tma_store_wait<0>();  // staging buffers stay valid until read
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *bail && a.err) atomicCAS(a.err, 0u, 0x47454d4du);
  if (UCCL_TIMES(a) && cta_id == 0 && threadIdx.x == 0) a.times[1] = ptx::globaltimer_ns();
  if (COMM == kCommReduceScatter && !*bail && !UCCL_DBG(a, 1)) {
    if (UCCL_DBG(a, 128)) reduce_scatter_tail_direct(a, cta_id, gemm_ctas);
    else reduce_scatter_tail(a, smem, bars + 24, bail, cta_id, gemm_ctas);
  }
}

// ------------------------------------------------------------------ CTA-pair kernel
// Two CTAs of a cluster share one 256 x 256 output tile (tcgen05 cta_group::2): each CTA stages
// its own 128 A rows and one half (128 rows) of the B tile, the leader CTA issues one MMA that
// reads both CTAs' shared memory, and each CTA's TMEM receives the accumulator rows of its own
// A rows.  Compared with the single-CTA kernel the B operand is fetched once per 256 output rows
// instead of once per 128, which cuts shared-memory fill traffic by a third and leaves room for
// six pipeline stages.
template <int EPI, int COMM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(COMM == kCommAllGather ? NUM_THREADS_FWD : NUM_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ PeerMaps pm, const Args a) {
  // The reduce-scatter fusion trades one pipeline stage for a deeper epilogue staging area: a
  // whole tile (4 x 4 KiB per warp) can be handed to the TMA without waiting for earlier stores,
  // which decouples the accumulator hand-back from the pace of the links.
  constexpr int ST = COMM == kCommReduceScatter ? pair::STAGES - 1 : pair::STAGES;
  constexpr int NBUF = COMM == kCommReduceScatter ? 4 : 2;
  constexpr int EPI_OFF = COMM == kCommReduceScatter ? ST * pair::STAGE_BYTES : PIPE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PIPE_BYTES + EPI_STAGE_BYTES);
  if (COMM == kCommAllGather && static_cast<int>(blockIdx.x) < a.comm_ctas) {
    if (!UCCL_DBG(a, 1) && threadIdx.x == 0 && wait_go(a.comm))
      comm_allgather_push<COPY_SLOT_BYTES, COPY_SLOTS, 4, 4>(a, smem, bars, blockIdx.x, a.comm_ctas);
    return;
  }
  const int cta_id = static_cast<int>(blockIdx.x) - a.comm_ctas;
  if (COMM == kCommReduceScatter && cta_id >= a.gemm_ctas) {
    // reducer CTA (both CTAs of such a cluster, independently): sums the staged copies of this
    // rank's row blocks as they complete, from the start of the launch
    volatile uint32_t* rbail = reinterpret_cast<volatile uint32_t*>(bars + 28);
    if (threadIdx.x == 0) *rbail = 0;
    __syncthreads();
    reduce_scatter_tail(a, smem, bars + 24, rbail, cta_id, a.gemm_ctas);
    return;
  }
  uint64_t* full_bar = bars;                           // [STAGES]  used in the leader
  uint64_t* empty_bar = bars + ST;           // [STAGES]  one per CTA
  uint64_t* tfull_bar = bars + 2 * ST;       // [2]       one per CTA
  uint64_t* tempty_bar = bars + 2 * ST + 2;  // [2]       used in the leader
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * ST + 4);
  volatile uint32_t* bail = tmem_holder + 1;
  uint32_t* warps_done = tmem_holder + 2;

  if (UCCL_TIMES(a) && cta_id == 0 && threadIdx.x == 0) a.times[0] = ptx::globaltimer_ns();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = ptx::cluster_ctarank();  // 0 = leader
  const bool leader = crank == 0;
  const int pairs = a.gemm_ctas / 2;
  const int pair_id = cta_id / 2;
  const int tiles_m2 = (a.M + 2 * BM - 1) / (2 * BM);
  const int num_tiles = tiles_m2 * a.tiles_n;
  const int num_kb = (a.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      ptx::mbar_init(&full_bar[s], 1);   // the leader's arrive.expect_tx; bytes come from both CTAs
      ptx::mbar_init(&empty_bar[s], 1);  // one tcgen05.commit from the leader
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&tfull_bar[i], 1);
      ptx::mbar_init(&tempty_bar[i], 8);  // four epilogue warps in each of the two CTAs
    }
    *bail = 0;
    warps_done[0] = warps_done[1] = warps_done[2] = warps_done[3] = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB);
    if (COMM == kCommAllGather) ptx::prefetch_tmap(&pm.m[0]);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_holder, TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // both CTAs' barriers and TMEM exist before anybody signals the other
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t full0 = ptx::mapa(ptx::smem_u32(&full_bar[0]), 0);
  const uint32_t tempty0 = ptx::mapa(ptx::smem_u32(&tempty_bar[0]), 0);
  const uint32_t empty_peer = ptx::mapa(ptx::smem_u32(&empty_bar[0]), 1);
  const uint32_t tfull_peer = ptx::mapa(ptx::smem_u32(&tfull_bar[0]), 1);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = pair_id; tile < num_tiles && !*bail; tile += pairs) {
        int mb2, nb;
        tile_coords<8>(a, tile, tiles_m2, 2, mb2, nb);
        const int mb = 2 * mb2 + static_cast<int>(crank);  // this CTA's 128-row block
        const bool own = mb >= a.a_local_lo && mb < a.a_local_hi;
        if (a.a_ready && !UCCL_DBG(a, 8) && !own) {
          if (!wait_flag_geq(a.a_ready + static_cast<size_t>(mb) * FLAG_STRIDE, a.a_ready_target, a.comm.timeout_ns,
                             a.comm.abort_flag)) {
            if (a.err) atomicCAS(a.err, 0u, 0x41470000u | static_cast<uint32_t>(mb));
            *bail = 1;
            break;
          }
          ptx::fence_proxy_async();  // the rows were written by bulk stores (async proxy)
        }
        // my own rows are read from the shard itself; pm.m[0] is its tensor map
        const bool fromShard = COMM == kCommAllGather && own && a.a_own_shard;
        const CUtensorMap* ta = fromShard ? &pm.m[0] : &tmA;
        const int m0 = fromShard ? (mb - a.a_local_lo) * BM : mb * BM;
        int brow;
        if (EPI == kEpiSwiGLU) brow = (leader ? 0 : a.b_half_rows) + nb * (BN / 2);  // gate | up
        else brow = nb * BN + static_cast<int>(crank) * (BN / 2);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % ST;
          const uint32_t ph = (it / ST) & 1;
          if (!ptx::mbar_wait_bounded(&empty_bar[s], ph ^ 1, bail)) break;
          uint8_t* sA = smem + s * pair::STAGE_BYTES;
          uint8_t* sB = sA + pair::A_BYTES;
          if (leader) ptx::mbar_expect_tx(&full_bar[s], 2 * pair::STAGE_BYTES);
          const uint32_t fb = full0 + static_cast<uint32_t>(s) * 8;
          ptx::tma_load_2d_pair(sA, ta, fb, kb * BK, m0);
          ptx::tma_load_2d_pair(sB, &tmB, fb, kb * BK, brow);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = ptx::umma_idesc_f16(1u, 2 * BM, BN);
      uint32_t it = 0, tcount = 0;
      for (int tile = pair_id; tile < num_tiles && !*bail; tile += pairs, ++tcount) {
        const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
        if (!ptx::mbar_wait_bounded(&tempty_bar[acc], acc_ph ^ 1, bail)) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % ST;
          const uint32_t ph = (it / ST) & 1;
          if (!ptx::mbar_wait_bounded(&full_bar[s], ph, bail)) break;
          ptx::tc_fence_after();
          const uint32_t sA = ptx::smem_u32(smem + s * pair::STAGE_BYTES);
          const uint64_t da = ptx::umma_smem_desc_sw128(sA);
          const uint64_t db = ptx::umma_smem_desc_sw128(sA + pair::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t koff = static_cast<uint64_t>((k * UMMA_K * 2) >> 4);
            ptx::umma_f16_pair(d_tmem, da + koff, db + koff, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          ptx::umma_commit_pair(ptx::smem_u32(&empty_bar[s]));
          ptx::umma_commit_pair(empty_peer + static_cast<uint32_t>(s) * 8);
        }
        ptx::umma_commit_pair(ptx::smem_u32(&tfull_bar[acc]));
        ptx::umma_commit_pair(tfull_peer + acc * 8);
      }
    } else if (COMM != kCommNone && a.comm.go && cta_id == 0) {
      prologue_barrier(a.comm, lane, a.err);  // the warp's idle lanes run the launch's rank barrier
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ forwarder (all-gather, spread mode)
    int go_ok = 1;
    if (COMM == kCommAllGather && a.a_spread && lane == 0) go_ok = wait_go(a.comm) ? 1 : 0;
    go_ok = __shfl_sync(0xffffffffu, go_ok, 0);
    if (COMM == kCommAllGather && a.a_spread && !UCCL_DBG(a, 1) && go_ok) {
      if (lane == 0) comm_allgather_push<FWD_SLOT_BYTES, FWD_SLOTS, 2, 2>(a, smem + PIPE_BYTES, bars + 24, blockIdx.x, gridDim.x);
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (both CTAs)
    const int q = warp & 3;
    uint8_t* stage = smem + EPI_OFF + q * NBUF * EPI_BUF_BYTES;
    uint32_t tcount = 0, stage_it = 0;
    int prev_mb = 0;
    if (COMM == kCommReduceScatter) {
      // no tile leaves for a peer before every rank has entered this launch
      int g = 1;
      if (lane == 0) g = wait_go(a.comm) ? 1 : 0;
      if (!__shfl_sync(0xffffffffu, g, 0) && lane == 0) *bail = 1;
      __syncwarp();
    }
    for (int tile = pair_id; tile < num_tiles && !*bail; tile += pairs, ++tcount) {
      int mb2, nb;
      tile_coords<8>(a, tile, tiles_m2, 2, mb2, nb);
      const int mb = 2 * mb2 + static_cast<int>(crank);
      const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
      if (!ptx::mbar_wait_bounded(&tfull_bar[acc], acc_ph, bail)) break;
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      epilogue_tile<EPI, COMM, NBUF>(a, pm, taddr, mb, nb, q, lane, stage, stage_it, a.C,
                                     a.epi_tma ? &pm.m[kMaxPeers] : nullptr, mb * BM + q * 32);
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(tempty0 + acc * 8);
      if (COMM == kCommReduceScatter) {
        if (tcount > 0) publish_tile<BN / 64>(a, prev_mb, lane, &warps_done[(tcount - 1) & 3]);
        prev_mb = mb;
      }
    }
    if (COMM == kCommReduceScatter && tcount > 0) publish_tile<0>(a, prev_mb, lane, &warps_done[(tcount - 1) & 3]);
    if (COMM != kCommReduceScatter && a.epi_tma && lane == 0) ptx::tma_store_wait<0>();  // staging buffers stay valid until read
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // nobody leaves while the other CTA may still signal it or read its memory
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *bail && a.err) atomicCAS(a.err, 0u, 0x47454d32u);
  if (UCCL_TIMES(a) && cta_id == 0 && threadIdx.x == 0) a.times[1] = ptx::globaltimer_ns();
  if (COMM == kCommReduceScatter && !*bail && !UCCL_DBG(a, 1)) {
    if (UCCL_DBG(a, 128)) reduce_scatter_tail_direct(a, cta_id, a.gemm_ctas);
    else reduce_scatter_tail(a, smem, bars + 24, bail, cta_id, a.gemm_ctas);
  }
}

}  // namespace gemm
}  // namespace uccl
