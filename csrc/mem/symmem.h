// Symmetric memory: every rank of an NVLink domain allocates the same amount, and maps every
// peer's allocation (plus, where the hardware has it, an NVSwitch multicast alias) into its own
// address space.  Kernels then reach peers with ordinary loads/stores and multimem.* on the
// multicast alias.
//
// This replaces the reference's Level-Zero IPC exchange (zeMemGetIpcHandle / MPI_Allgather /
// zeMemOpenIpcHandle in src/rma/rma.cc:78-152 and the never-opened handle of
// src/transport/p2p.cc:48-104).  Preferred mechanism: CUDA VMM -- cuMemCreate with a POSIX file
// descriptor handle type, descriptors passed between processes with SCM_RIGHTS, cuMemMap +
// cuMemSetAccess on the importer, cuMulticastCreate/AddDevice/BindMem for the NVLS alias.
// Fallback: cudaMalloc + cudaIpc handles (no multicast).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <vector>

#include "../core/bootstrap.h"
#include "../core/config.h"
#include "uccl.h"

namespace uccl {

enum SymMode : int { SYM_NONE = 0, SYM_IPC = 1, SYM_VMM = 2 };

struct SymSegment {
  char* local = nullptr;
  size_t size = 0;     // bytes the caller asked for
  size_t mapSize = 0;  // bytes actually mapped (granularity multiple)
  size_t guard = 0;    // canary bytes in front of the caller's pointer (0 = no canaries), see ucclMemCheck
  size_t userSize = 0; // bytes between the two canaries
  char* peer[UCCL_MAX_LOCAL_RANKS] = {};
  char* mc = nullptr;  // multicast alias or nullptr
  int mode = SYM_NONE;
  CUmemGenericAllocationHandle handle = 0;
  CUmemGenericAllocationHandle peerHandle[UCCL_MAX_LOCAL_RANKS] = {};
  CUmemGenericAllocationHandle mcHandle = 0;
  bool mcBound = false;
};

class SymHeap {
 public:
  // localGlobalRanks[i] = communicator rank of NVLink-domain member i.
  ucclResult_t init(Bootstrap* bs, const std::vector<int>& localGlobalRanks, int localRank, int cudaDev,
                    const Config& cfg);
  // Collective over the whole communicator (ranks outside this domain run their own domain).
  ucclResult_t alloc(size_t size, SymSegment** out);
  ucclResult_t release(SymSegment* seg);
  void releaseAll();
  // Segment that contains [ptr, ptr + bytes), or nullptr.
  SymSegment* find(const void* ptr, size_t bytes);
  std::vector<SymSegment*> segments();  // snapshot of the live segments

  int mode() const { return mode_; }
  bool nvls() const { return nvls_; }
  int localRank() const { return localRank_; }
  int localRanks() const { return static_cast<int>(ranks_.size()); }

 private:
  ucclResult_t allocVmm(size_t size, SymSegment* seg);
  ucclResult_t allocIpc(size_t size, SymSegment* seg);
  bool agree(bool mine);  // true iff every local rank passed true

  Bootstrap* bs_ = nullptr;
  std::vector<int> ranks_;
  int localRank_ = 0;
  int dev_ = 0;
  int mode_ = SYM_NONE;
  bool nvls_ = false;
  int seq_ = 0;
  std::mutex mu_;
  std::vector<SymSegment*> segs_;
};

}  // namespace uccl
