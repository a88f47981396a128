#include "symmem.h"

#include <string.h>
#include <unistd.h>

#include <algorithm>

#include "../core/cuda_driver.h"
#include "../core/log.h"

namespace uccl {

namespace {
constexpr int kFdTagBase = 1000;   // tag space for allocation handles
constexpr int kMcTagBase = 500000; // tag space for multicast handles

size_t roundUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

#define CU_TRY(call, onfail)                                                               \
  do {                                                                                     \
    CUresult _r = (call);                                                                  \
    if (_r != CUDA_SUCCESS) {                                                              \
      UCCL_LOG(WARN, "%s failed: %s", #call, driverErrorString(_r));                       \
      onfail;                                                                              \
    }                                                                                      \
  } while (0)
}  // namespace

ucclResult_t SymHeap::init(Bootstrap* bs, const std::vector<int>& localGlobalRanks, int localRank, int cudaDev,
                           const Config& cfg) {
  bs_ = bs;
  ranks_ = localGlobalRanks;
  localRank_ = localRank;
  dev_ = cudaDev;
  const DriverApi& d = driverApi();
  if (static_cast<int>(ranks_.size()) > UCCL_MAX_LOCAL_RANKS) return ucclInvalidArgument;

  bool vmmOk = d.ok && cfg.p2pMode != 1;
  if (vmmOk) {
    int v = 0;
    CUdevice cd;
    if (d.deviceGet(&cd, dev_) != CUDA_SUCCESS ||
        d.deviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cd) != CUDA_SUCCESS ||
        !v)
      vmmOk = false;
  }
  bool mcOk = vmmOk && cfg.nvls != 0 && d.multicastCreate && ranks_.size() > 1;
  if (mcOk) {
    int v = 0;
    CUdevice cd;
    d.deviceGet(&cd, dev_);
    if (d.deviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) != CUDA_SUCCESS || !v) mcOk = false;
  }
  // every member of the domain must take the same path
  vmmOk = agree(vmmOk);
  mcOk = agree(mcOk) && vmmOk;
  mode_ = vmmOk ? SYM_VMM : SYM_IPC;
  nvls_ = mcOk;
  if (cfg.nvls == 1 && !nvls_) {
    UCCL_LOG(ERROR, "UCCL_NVLS=1 but multicast objects are not available on every rank");
    return ucclSystemError;
  }
  UCCL_LOG(INFO, "symmetric heap: mode=%s nvls=%d domain=%zu", mode_ == SYM_VMM ? "vmm" : "ipc", (int)nvls_,
           ranks_.size());
  return ucclSuccess;
}

bool SymHeap::agree(bool mine) {
  const int n = bs_->nranks();
  if (n <= 1) return mine;
  std::vector<uint8_t> v(n, 0);
  v[bs_->rank()] = mine ? 1 : 0;
  if (bs_->allGather(v.data(), 1) != ucclSuccess) return false;
  for (int r : ranks_)
    if (!v[r]) return false;
  return true;
}

ucclResult_t SymHeap::alloc(size_t size, SymSegment** out) {
  if (!out || size == 0) return ucclInvalidArgument;
  SymSegment* seg = new SymSegment();
  seg->size = size;
  ucclResult_t r = (mode_ == SYM_VMM) ? allocVmm(size, seg) : allocIpc(size, seg);
  if (r != ucclSuccess) {
    delete seg;
    return r;
  }
  ++seq_;
  std::lock_guard<std::mutex> lk(mu_);
  segs_.push_back(seg);
  *out = seg;
  return ucclSuccess;
}

ucclResult_t SymHeap::allocVmm(size_t size, SymSegment* seg) {
  const DriverApi& d = driverApi();
  const int n = static_cast<int>(ranks_.size());
  seg->mode = SYM_VMM;

  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 2u << 20;
  CU_TRY(d.memGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), gran = 2u << 20);

  CUmulticastObjectProp mcProp;
  memset(&mcProp, 0, sizeof(mcProp));
  bool wantMc = nvls_;
  if (wantMc) {
    mcProp.numDevices = n;
    mcProp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mcProp.size = roundUp(size, gran);
    size_t mcGran = 0;
    if (d.multicastGetGranularity(&mcGran, &mcProp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mcGran)
      gran = std::max(gran, mcGran);
  }
  const size_t mapSize = roundUp(size, gran);
  seg->mapSize = mapSize;
  mcProp.size = mapSize;

  bool ok = true;
  UCCL_LOG(TRACE, "symmem: cuMemCreate %zu bytes (granularity %zu)", mapSize, gran);
  CU_TRY(d.memCreate(&seg->handle, mapSize, &prop, 0), ok = false);
  if (!agree(ok)) {
    if (ok) d.memRelease(seg->handle);
    UCCL_LOG(ERROR, "symmetric allocation of %zu bytes failed on some rank", mapSize);
    return ucclSystemError;
  }

  CUmemAccessDesc access;
  memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = dev_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;

  auto mapHandle = [&](CUmemGenericAllocationHandle h, char** va) -> bool {
    CUdeviceptr p = 0;
    if (d.memAddressReserve(&p, mapSize, gran, 0, 0) != CUDA_SUCCESS) return false;
    if (d.memMap(p, mapSize, 0, h, 0) != CUDA_SUCCESS) {
      d.memAddressFree(p, mapSize);
      return false;
    }
    if (d.memSetAccess(p, mapSize, &access, 1) != CUDA_SUCCESS) {
      d.memUnmap(p, mapSize);
      d.memAddressFree(p, mapSize);
      return false;
    }
    *va = reinterpret_cast<char*>(p);
    return true;
  };

  ok = mapHandle(seg->handle, &seg->local);
  seg->peer[localRank_] = seg->local;

  // exchange allocation handles as file descriptors
  int myFd = -1;
  if (n > 1) {
    CU_TRY(d.memExportToShareableHandle(&myFd, seg->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), ok = false);
    const int tag = kFdTagBase + seq_;
    if (ok)
      for (int i = 0; i < n; ++i) {
        if (i == localRank_) continue;
        if (bs_->sendFd(ranks_[i], tag, myFd) != ucclSuccess) ok = false;
      }
    if (ok)
      for (int i = 0; i < n && ok; ++i) {
        if (i == localRank_) continue;
        int fd = -1;
        if (bs_->recvFd(ranks_[i], tag, &fd) != ucclSuccess) {
          ok = false;
          break;
        }
        CUresult ir = d.memImportFromShareableHandle(&seg->peerHandle[i], reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                     CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        ::close(fd);
        if (ir != CUDA_SUCCESS) {
          UCCL_LOG(WARN, "cuMemImportFromShareableHandle (peer %d): %s", i, driverErrorString(ir));
          ok = false;
          break;
        }
        if (!mapHandle(seg->peerHandle[i], &seg->peer[i])) ok = false;
      }
  }
  UCCL_LOG(TRACE, "symmem: peer handles mapped ok=%d", (int)ok);
  // keep myFd open until every peer imported it
  const bool allOk = agree(ok);
  if (myFd >= 0) ::close(myFd);
  if (!allOk) {
    UCCL_LOG(ERROR, "symmetric mapping failed on some rank");
    return ucclSystemError;
  }

  // NVSwitch multicast alias
  if (wantMc) {
    bool mok = true;
    int mcFd = -1;
    const int tag = kMcTagBase + seq_;
    if (localRank_ == 0) {
      CU_TRY(d.multicastCreate(&seg->mcHandle, &mcProp), mok = false);
      if (mok) CU_TRY(d.memExportToShareableHandle(&mcFd, seg->mcHandle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), mok = false);
    }
    // rank 0 tells the others whether an fd is coming
    mok = agree(mok);
    if (mok) {
      if (localRank_ == 0) {
        for (int i = 1; i < n; ++i)
          if (bs_->sendFd(ranks_[i], tag, mcFd) != ucclSuccess) mok = false;
      } else {
        int fd = -1;
        if (bs_->recvFd(ranks_[0], tag, &fd) != ucclSuccess) mok = false;
        if (mok) {
          CU_TRY(d.memImportFromShareableHandle(&seg->mcHandle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                 mok = false);
          ::close(fd);
        }
      }
    }
    mok = agree(mok);
    if (mcFd >= 0) ::close(mcFd);
    if (mok) CU_TRY(d.multicastAddDevice(seg->mcHandle, dev_), mok = false);
    UCCL_LOG(TRACE, "symmem: multicast device added ok=%d", (int)mok);
    mok = agree(mok);  // every device must be added before anybody binds
    if (mok) {
      CU_TRY(d.multicastBindMem(seg->mcHandle, 0, seg->handle, 0, mapSize, 0), mok = false);
      if (mok) seg->mcBound = true;
    }
    UCCL_LOG(TRACE, "symmem: multicast bound ok=%d", (int)mok);
    mok = agree(mok);
    if (mok) {
      if (!mapHandle(seg->mcHandle, &seg->mc)) mok = false;
    }
    mok = agree(mok);
    if (!mok) {
      UCCL_LOG(WARN, "multicast binding failed; segment of %zu bytes continues without NVLS", mapSize);
      if (seg->mc) {
        d.memUnmap(reinterpret_cast<CUdeviceptr>(seg->mc), mapSize);
        d.memAddressFree(reinterpret_cast<CUdeviceptr>(seg->mc), mapSize);
        seg->mc = nullptr;
      }
      if (seg->mcBound && d.multicastUnbind) d.multicastUnbind(seg->mcHandle, dev_, 0, mapSize);
      seg->mcBound = false;
      if (seg->mcHandle) d.memRelease(seg->mcHandle);
      seg->mcHandle = 0;
      nvls_ = false;  // one failure disables NVLS for the communicator: all ranks agree on it
    }
  }
  return ucclSuccess;
}

ucclResult_t SymHeap::allocIpc(size_t size, SymSegment* seg) {
  const int n = static_cast<int>(ranks_.size());
  seg->mode = SYM_IPC;
  seg->mapSize = roundUp(size, 2u << 20);
  void* p = nullptr;
  bool ok = cudaMalloc(&p, seg->mapSize) == cudaSuccess;
  if (!ok) (void)cudaGetLastError();
  seg->local = static_cast<char*>(p);
  seg->peer[localRank_] = seg->local;
  if (n > 1) {
    const int world = bs_->nranks();
    std::vector<cudaIpcMemHandle_t> hs(world);
    memset(hs.data(), 0, sizeof(cudaIpcMemHandle_t) * world);
    if (ok && cudaIpcGetMemHandle(&hs[bs_->rank()], p) != cudaSuccess) {
      (void)cudaGetLastError();
      ok = false;
    }
    if (bs_->allGather(hs.data(), sizeof(cudaIpcMemHandle_t)) != ucclSuccess) ok = false;
    if (ok)
      for (int i = 0; i < n; ++i) {
        if (i == localRank_) continue;
        void* pp = nullptr;
        if (cudaIpcOpenMemHandle(&pp, hs[ranks_[i]], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
          UCCL_LOG(WARN, "cudaIpcOpenMemHandle (peer %d): %s", i, cudaGetErrorString(cudaGetLastError()));
          ok = false;
          break;
        }
        seg->peer[i] = static_cast<char*>(pp);
      }
  }
  if (!agree(ok)) {
    UCCL_LOG(ERROR, "cudaIpc symmetric allocation failed on some rank");
    return ucclSystemError;
  }
  return ucclSuccess;
}

SymSegment* SymHeap::find(const void* ptr, size_t bytes) {
  const char* p = static_cast<const char*>(ptr);
  std::lock_guard<std::mutex> lk(mu_);
  for (SymSegment* s : segs_)
    if (p >= s->local && p + bytes <= s->local + s->mapSize) return s;
  return nullptr;
}

std::vector<SymSegment*> SymHeap::segments() {
  std::lock_guard<std::mutex> lk(mu_);
  return segs_;
}

ucclResult_t SymHeap::release(SymSegment* seg) {
  if (!seg) return ucclInvalidArgument;
  {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = std::find(segs_.begin(), segs_.end(), seg);
    if (it == segs_.end()) return ucclInvalidArgument;
    segs_.erase(it);
  }
  const DriverApi& d = driverApi();
  const int n = static_cast<int>(ranks_.size());
  if (seg->mode == SYM_VMM) {
    if (seg->mc) {
      d.memUnmap(reinterpret_cast<CUdeviceptr>(seg->mc), seg->mapSize);
      d.memAddressFree(reinterpret_cast<CUdeviceptr>(seg->mc), seg->mapSize);
    }
    if (seg->mcBound && d.multicastUnbind) d.multicastUnbind(seg->mcHandle, dev_, 0, seg->mapSize);
    if (seg->mcHandle) d.memRelease(seg->mcHandle);
    for (int i = 0; i < n; ++i) {
      if (!seg->peer[i]) continue;
      d.memUnmap(reinterpret_cast<CUdeviceptr>(seg->peer[i]), seg->mapSize);
      d.memAddressFree(reinterpret_cast<CUdeviceptr>(seg->peer[i]), seg->mapSize);
      if (i != localRank_ && seg->peerHandle[i]) d.memRelease(seg->peerHandle[i]);
    }
    if (seg->handle) d.memRelease(seg->handle);
  } else if (seg->mode == SYM_IPC) {
    for (int i = 0; i < n; ++i)
      if (i != localRank_ && seg->peer[i]) cudaIpcCloseMemHandle(seg->peer[i]);
    if (seg->local) cudaFree(seg->local);
  }
  delete seg;
  return ucclSuccess;
}

void SymHeap::releaseAll() {
  while (true) {
    SymSegment* s = nullptr;
    {
      std::lock_guard<std::mutex> lk(mu_);
      if (segs_.empty()) break;
      s = segs_.back();
    }
    release(s);
  }
}

}  // namespace uccl
