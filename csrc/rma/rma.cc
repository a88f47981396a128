#include "rma.h"

#include <string.h>

#include <algorithm>

#include "../core/cuda_driver.h"
#include "../core/enqueue.h"
#include "../core/log.h"
#include "rma_kernels.h"

using namespace uccl;

namespace uccl {

namespace {

bool winValid(const Window* w) { return w && w->magic == 0x57494e44 && commValid(w->comm); }

void closeWindow(Window* w) {
  Comm* c = w->comm;
  for (int p = 0; p < c->localRanks; ++p)
    if (w->ipcOpened[p] && w->ipcBase[p]) cudaIpcCloseMemHandle(w->ipcBase[p]);
  if (w->dynTables) cudaFree(w->dynTables);
  w->magic = 0;
  delete w;
}

struct DeviceGuard {
  int prev = -1, want;
  explicit DeviceGuard(int dev) : want(dev) {
    cudaGetDevice(&prev);
    if (prev != want) cudaSetDevice(want);
  }
  ~DeviceGuard() {
    if (prev >= 0 && prev != want) cudaSetDevice(prev);
  }
};

struct IpcBlob {
  cudaIpcMemHandle_t handle;
  uint64_t offset;    // of the window inside the allocation the handle names
  uint64_t symOffset; // offset inside a symmetric segment, or ~0
  int32_t symmetric;
  int32_t valid;
};

ucclResult_t checkXfer(Window* w, Comm* c, const void* local, size_t count, ucclDataType_t dt, int peer, size_t off,
                       size_t* bytes) {
  if (!winValid(w) || w->comm != c) return ucclInvalidArgument;
  if (dt < 0 || dt >= ucclNumTypes) return ucclInvalidArgument;
  if (peer < 0 || peer >= c->nRanks || peer == c->rank) return ucclInvalidArgument;
  if (count && !local) return ucclInvalidArgument;
  *bytes = count * dataTypeSize(dt);
  if (off > w->size || *bytes > w->size - off) return ucclInvalidArgument;
  return ucclSuccess;
}

ucclResult_t copyAndSignal(Comm* c, char* dst, const char* src, size_t bytes, uint64_t* signal, cudaStream_t s) {
  cudaError_t e = cudaSuccess;
  if (bytes > (8u << 20)) {
    // large transfers ride a copy engine, the signal follows in stream order
    e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s);
    if (e == cudaSuccess && signal) e = launchRmaSignal(signal, s);
  } else if (bytes > 0 || signal) {
    e = launchRmaCopySignal(dst, src, bytes, signal, c->epochsDev + kMaxBlocks + kLLBlocks, s);
  }
  if (e != cudaSuccess) {
    commSetError(c, "RMA launch failed: %s", cudaGetErrorString(e));
    return ucclSystemError;
  }
  return ucclSuccess;
}

}  // namespace

void rmaDestroyAll(Comm* c) {
  std::lock_guard<std::mutex> lk(c->winMu);
  for (Window* w : c->windows)
    if (w) closeWindow(w);
  c->windows.clear();
}

}  // namespace uccl

extern "C" ucclResult_t ucclCommWindowRegister(ucclWindow_t* win, void* buff, size_t size, ucclComm_t comm) {
  Comm* c = toComm(comm);
  if (!commValid(c) || !win || !buff || size == 0) return ucclInvalidArgument;
  *win = nullptr;
  if (c->backend != BACKEND_CUDA || !c->p2pReady) {
    commSetError(c, "windows need ranks that share an NVLink domain");
    return ucclInvalidUsage;
  }
  DeviceGuard guard(c->cudaDev);
  int slot = -1;
  {
    std::lock_guard<std::mutex> lk(c->winMu);
    for (size_t i = 0; i < c->windows.size(); ++i)
      if (!c->windows[i]) { slot = static_cast<int>(i); break; }
    if (slot < 0 && c->windows.size() < static_cast<size_t>(kMaxWindows)) {
      slot = static_cast<int>(c->windows.size());
      c->windows.push_back(nullptr);
    }
  }
  if (slot < 0) {
    commSetError(c, "too many windows (limit %d)", kMaxWindows);
    return ucclInvalidUsage;
  }
  Window* w = new Window();
  w->comm = c;
  w->slot = slot;
  w->localBuff = static_cast<char*>(buff);
  w->size = size;
  const size_t sigOff = kArenaWinSignalOff + static_cast<size_t>(slot) * UCCL_MAX_LOCAL_RANKS * sizeof(uint64_t);
  w->localSignals = reinterpret_cast<uint64_t*>(c->arena->local + sigOff);
  for (int p = 0; p < c->localRanks; ++p) w->remoteSignals[p] = reinterpret_cast<uint64_t*>(c->arena->peer[p] + sigOff);
  cudaMemsetAsync(w->localSignals, 0, UCCL_MAX_LOCAL_RANKS * sizeof(uint64_t), nullptr);
  cudaStreamSynchronize(nullptr);

  // how can peers reach this buffer?
  std::vector<IpcBlob> blobs(c->nRanks);
  memset(blobs.data(), 0, sizeof(IpcBlob) * c->nRanks);
  IpcBlob& mine = blobs[c->rank];
  SymSegment* seg = c->heap.find(buff, size);
  if (seg) {
    mine.symmetric = 1;
    mine.symOffset = static_cast<uint64_t>(static_cast<char*>(buff) - seg->local);
    mine.valid = 1;
  } else {
    cudaError_t e = cudaIpcGetMemHandle(&mine.handle, buff);
    if (e == cudaSuccess) {
      // the handle names the whole allocation; find where the window starts inside it
      CUdeviceptr base = 0;
      size_t range = 0;
      const DriverApi& d = driverApi();
      if (d.ok && d.memGetAddressRange(&base, &range, reinterpret_cast<CUdeviceptr>(buff)) == CUDA_SUCCESS && base) {
        mine.offset = static_cast<uint64_t>(reinterpret_cast<CUdeviceptr>(buff) - base);
        mine.valid = 1;
      }
    } else {
      (void)cudaGetLastError();
    }
  }
  ucclResult_t r = c->bootstrap.allGather(blobs.data(), sizeof(IpcBlob));
  bool ok = r == ucclSuccess;
  for (int p = 0; ok && p < c->localRanks; ++p) {
    const int gr = c->localGlobalRanks[p];
    const IpcBlob& b = blobs[gr];
    if (gr == c->rank) {
      w->remotePtrs[p] = w->localBuff;
      continue;
    }
    if (!b.valid) { ok = false; break; }
    if (b.symmetric) {
      // symmetric convention: the same segment order on every rank, so the segment that holds my
      // buffer at this offset is the one that holds the peer's
      if (!seg) { ok = false; break; }
      w->remotePtrs[p] = seg->peer[p] + b.symOffset;
    } else {
      void* base = nullptr;
      if (cudaIpcOpenMemHandle(&base, b.handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        (void)cudaGetLastError();
        ok = false;
        break;
      }
      w->ipcOpened[p] = true;
      w->ipcBase[p] = static_cast<char*>(base);
      w->remotePtrs[p] = static_cast<char*>(base) + b.offset;
    }
  }
  // all ranks succeed or all fail
  std::vector<uint8_t> flags(c->nRanks, 0);
  flags[c->rank] = ok ? 1 : 0;
  if (c->bootstrap.allGather(flags.data(), 1) != ucclSuccess) ok = false;
  for (uint8_t f : flags)
    if (!f) ok = false;
  if (!ok) {
    commSetError(c, "window registration failed: the buffer cannot be mapped by every peer "
                    "(allocate it with ucclMemAlloc, or with cudaMalloc in a separate process per rank)");
    closeWindow(w);
    std::lock_guard<std::mutex> lk(c->winMu);
    c->windows[slot] = nullptr;
    return ucclSystemError;
  }
  {
    std::lock_guard<std::mutex> lk(c->winMu);
    c->windows[slot] = w;
  }
  *win = reinterpret_cast<ucclWindow_t>(w);
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommWindowDeregister(ucclWindow_t win) {
  Window* w = reinterpret_cast<Window*>(win);
  if (!w) return ucclSuccess;
  if (!winValid(w)) return ucclInvalidArgument;
  Comm* c = w->comm;
  DeviceGuard guard(c->cudaDev);
  cudaDeviceSynchronize();
  c->bootstrap.barrier();  // nobody is still writing into this window
  {
    std::lock_guard<std::mutex> lk(c->winMu);
    if (w->slot >= 0 && w->slot < static_cast<int>(c->windows.size())) c->windows[w->slot] = nullptr;
  }
  closeWindow(w);
  return ucclSuccess;
}

extern "C" ucclResult_t ucclPut(const void* localBuff, size_t count, ucclDataType_t datatype, int peer,
                                ucclWindow_t peerWin, size_t peerWinOffset, ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  Window* w = reinterpret_cast<Window*>(peerWin);
  size_t bytes = 0;
  ucclResult_t r = checkXfer(w, c, localBuff, count, datatype, peer, peerWinOffset, &bytes);
  if (r != ucclSuccess) return r;
  UCCL_LOG(TRACE, "ucclPut peer=%d bytes=%zu off=%zu", peer, bytes, peerWinOffset);
  if (bytes == 0) return ucclSuccess;
  DeviceGuard guard(c->cudaDev);
  commCount(c, ucclCollRma, bytes, ucclAlgoAuto);
  const int lp = c->peers[peer].localRank;
  return copyAndSignal(c, w->remotePtrs[lp] + peerWinOffset, static_cast<const char*>(localBuff), bytes, nullptr,
                       static_cast<cudaStream_t>(stream));
}

extern "C" ucclResult_t ucclGet(void* localBuff, size_t count, ucclDataType_t datatype, int peer, ucclWindow_t peerWin,
                                size_t peerWinOffset, ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  Window* w = reinterpret_cast<Window*>(peerWin);
  size_t bytes = 0;
  ucclResult_t r = checkXfer(w, c, localBuff, count, datatype, peer, peerWinOffset, &bytes);
  if (r != ucclSuccess) return r;
  UCCL_LOG(TRACE, "ucclGet peer=%d bytes=%zu off=%zu", peer, bytes, peerWinOffset);
  if (bytes == 0) return ucclSuccess;
  DeviceGuard guard(c->cudaDev);
  commCount(c, ucclCollRma, bytes, ucclAlgoAuto);
  const int lp = c->peers[peer].localRank;
  return copyAndSignal(c, static_cast<char*>(localBuff), w->remotePtrs[lp] + peerWinOffset, bytes, nullptr,
                       static_cast<cudaStream_t>(stream));
}

extern "C" ucclResult_t ucclPutSignal(const void* localBuff, size_t count, ucclDataType_t datatype, int peer,
                                      ucclWindow_t peerWin, size_t peerWinOffset, int sigIdx, int ctx,
                                      unsigned int flags, ucclComm_t comm, void* stream) {
  (void)flags;
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  if (sigIdx != 0 || ctx != 0) return ucclInvalidArgument;
  Window* w = reinterpret_cast<Window*>(peerWin);
  size_t bytes = 0;
  ucclResult_t r = checkXfer(w, c, localBuff, count, datatype, peer, peerWinOffset, &bytes);
  if (r != ucclSuccess) return r;
  UCCL_LOG(TRACE, "ucclPutSignal peer=%d bytes=%zu off=%zu", peer, bytes, peerWinOffset);
  DeviceGuard guard(c->cudaDev);
  commCount(c, ucclCollRma, bytes, ucclAlgoAuto);
  const int lp = c->peers[peer].localRank;
  // the counter the peer keeps for me: remoteSignals[peer][my rank]
  return copyAndSignal(c, w->remotePtrs[lp] + peerWinOffset, static_cast<const char*>(localBuff), bytes,
                       w->remoteSignals[lp] + c->localRank, static_cast<cudaStream_t>(stream));
}

extern "C" ucclResult_t ucclGetSignal(void* localBuff, size_t count, ucclDataType_t datatype, int peer,
                                      ucclWindow_t peerWin, size_t peerWinOffset, int sigIdx, int ctx,
                                      unsigned int flags, ucclComm_t comm, void* stream) {
  (void)flags;
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  if (sigIdx != 0 || ctx != 0) return ucclInvalidArgument;
  Window* w = reinterpret_cast<Window*>(peerWin);
  size_t bytes = 0;
  ucclResult_t r = checkXfer(w, c, localBuff, count, datatype, peer, peerWinOffset, &bytes);
  if (r != ucclSuccess) return r;
  UCCL_LOG(TRACE, "ucclGetSignal peer=%d bytes=%zu off=%zu", peer, bytes, peerWinOffset);
  DeviceGuard guard(c->cudaDev);
  commCount(c, ucclCollRma, bytes, ucclAlgoAuto);
  const int lp = c->peers[peer].localRank;
  // completion marker on this rank: localSignals[peer]
  return copyAndSignal(c, static_cast<char*>(localBuff), w->remotePtrs[lp] + peerWinOffset, bytes,
                       w->localSignals + lp, static_cast<cudaStream_t>(stream));
}

extern "C" ucclResult_t ucclSignal(int peer, int sigIdx, int ctx, unsigned int flags, ucclComm_t comm, void* stream) {
  (void)flags;
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  if (sigIdx != 0 || ctx != 0) return ucclInvalidArgument;
  if (peer < 0 || peer >= c->nRanks || peer == c->rank) return ucclInvalidArgument;
  Window* w = nullptr;
  {
    std::lock_guard<std::mutex> lk(c->winMu);
    for (auto it = c->windows.rbegin(); it != c->windows.rend() && !w; ++it) w = *it;
  }
  if (!w) {
    commSetError(c, "ucclSignal needs a registered window to carry the counter");
    return ucclInvalidUsage;
  }
  UCCL_LOG(TRACE, "ucclSignal peer=%d window=%d", peer, w->slot);
  DeviceGuard guard(c->cudaDev);
  const int lp = c->peers[peer].localRank;
  if (launchRmaSignal(w->remoteSignals[lp] + c->localRank, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    commSetError(c, "signal kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  return ucclSuccess;
}

extern "C" ucclResult_t ucclWaitSignal(int nDesc, ucclWaitSignalDesc_t* signalDescs, ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  if (nDesc < 0 || nDesc > 8 || (nDesc && !signalDescs)) return ucclInvalidArgument;
  if (nDesc == 0) return ucclSuccess;
  RmaWaitArgs a;
  memset(&a, 0, sizeof(a));
  a.dc = c->dev;
  a.n = nDesc;
  for (int i = 0; i < nDesc; ++i) {
    const ucclWaitSignalDesc_t& d = signalDescs[i];
    Window* w = reinterpret_cast<Window*>(d.win);
    if (!winValid(w) || w->comm != c) return ucclInvalidArgument;
    if (d.sigIdx != 0 || d.ctx != 0 || d.opCnt < 0) return ucclInvalidArgument;
    if (d.peer < 0 || d.peer >= c->nRanks) return ucclInvalidArgument;
    const int lp = c->peers[d.peer].localRank;
    a.signals[i] = w->localSignals + lp;
    a.expected[i] = static_cast<uint64_t>(d.opCnt);
    a.peers[i] = d.peer;
  }
  UCCL_LOG(TRACE, "ucclWaitSignal n=%d", nDesc);
  DeviceGuard guard(c->cudaDev);
  if (launchRmaWait(a, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    commSetError(c, "wait kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  return ucclSuccess;
}

extern "C" ucclResult_t ucclWindowGetDeviceHandle(ucclWindow_t win, ucclDeviceWindow* out) {
  Window* w = reinterpret_cast<Window*>(win);
  if (!winValid(w) || !out) return ucclInvalidArgument;
  Comm* c = w->comm;
  memset(out, 0, sizeof(*out));
  out->localBuff = w->localBuff;
  out->size = w->size;
  out->nRanks = c->localRanks;
  out->myRank = c->localRank;
  out->localSignals = reinterpret_cast<unsigned long long*>(w->localSignals);
  out->timeoutNs = c->cfg.waitTimeoutMs * 1000000ull;
  for (int p = 0; p < c->localRanks; ++p) {
    out->remotePtrs[p] = w->remotePtrs[p];
    out->remoteSignals[p] = reinterpret_cast<unsigned long long*>(w->remoteSignals[p]);
  }
  return ucclSuccess;
}

// Pointer-table form of the descriptor (the reference's ucclDeviceWindowDyn,
// src/rma/rma_device.hpp:61-70): the two per-peer tables are copied to device memory once per
// window and freed with it.
extern "C" ucclResult_t ucclWindowGetDeviceHandleDyn(ucclWindow_t win, ucclDeviceWindowDyn* out) {
  Window* w = reinterpret_cast<Window*>(win);
  if (!winValid(w) || !out) return ucclInvalidArgument;
  Comm* c = w->comm;
  DeviceGuard guard(c->cudaDev);
  const int n = c->localRanks;
  {
    std::lock_guard<std::mutex> lk(c->winMu);
    if (!w->dynTables) {
      void* host[2 * UCCL_MAX_LOCAL_RANKS] = {};
      for (int p = 0; p < n; ++p) {
        host[p] = w->remotePtrs[p];
        host[UCCL_MAX_LOCAL_RANKS + p] = w->remoteSignals[p];
      }
      void* d = nullptr;
      if (cudaMalloc(&d, sizeof(host)) != cudaSuccess ||
          cudaMemcpy(d, host, sizeof(host), cudaMemcpyHostToDevice) != cudaSuccess) {
        if (d) cudaFree(d);
        (void)cudaGetLastError();
        commSetError(c, "no device memory for the window's pointer tables");
        return ucclSystemError;
      }
      w->dynTables = d;
    }
  }
  memset(out, 0, sizeof(*out));
  out->localBuff = w->localBuff;
  out->size = w->size;
  out->nRanks = n;
  out->myRank = c->localRank;
  out->localSignals = reinterpret_cast<unsigned long long*>(w->localSignals);
  out->timeoutNs = c->cfg.waitTimeoutMs * 1000000ull;
  out->remotePtrs = static_cast<char**>(w->dynTables);
  out->remoteSignals = reinterpret_cast<unsigned long long**>(static_cast<void**>(w->dynTables) + UCCL_MAX_LOCAL_RANKS);
  return ucclSuccess;
}
