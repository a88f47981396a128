#include <dlfcn.h>
// Communicator lifecycle.  Follows the order of the reference's ucclCommInitRank
// (src/init.cc:67-167: bootstrap -> plugin -> peer-info all-gather -> node count -> channels ->
// proxy) and of its teardown (src/init.cc:210-240), but every resource the reference leaves as a
// null pointer (device, queue, topology, symmetric context) is really created here, the unique id
// is honoured, and the caller's rank/size are authoritative.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <functional>
#include <set>
#include <thread>

#include "../rma/rma.h"
#include "comm.h"
#include "../kernels/device_comm.h"
#include "../transport/net_plugin.h"
#include "cuda_driver.h"
#include "log.h"
#include "trace.h"

namespace uccl {

uint64_t getHostHash() {
  char name[256] = {0};
  gethostname(name, sizeof(name) - 1);
  // include the boot id so that two containers with the same hostname on different machines differ
  std::string s(name);
  FILE* f = fopen("/proc/sys/kernel/random/boot_id", "r");
  if (f) {
    char buf[64] = {0};
    if (fgets(buf, sizeof(buf), f)) s += buf;
    fclose(f);
  }
  return std::hash<std::string>()(s);
}
uint64_t getPidHash() { return static_cast<uint64_t>(getpid()); }

size_t dataTypeSize(ucclDataType_t t) {
  switch (t) {
    case ucclFloat16:
    case ucclBfloat16: return 2;
    case ucclFloat32: return 4;
    case ucclFloat8e4m3:
    case ucclUint8: return 1;
    default: return 0;
  }
}

bool commValid(const Comm* c) { return c && c->magic == 0x55434c43; }

void commSetError(Comm* c, const char* fmt, ...) {
  char msg[256];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  UCCL_LOG(ERROR, "%s", msg);
  if (!c) return;
  std::lock_guard<std::mutex> lk(c->errMu);
  snprintf(c->lastError, sizeof(c->lastError), "%s", msg);
}

void commSetAsyncError(Comm* c, ucclResult_t r) {
  int expected = ucclSuccess;
  c->asyncError.compare_exchange_strong(expected, static_cast<int>(r));
}

void commCount(Comm* c, ucclCollKind_t kind, size_t bytes, ucclAlgo_t algo) {
  std::lock_guard<std::mutex> lk(c->ctrMu);
  c->counters.ops[kind]++;
  c->counters.bytes[kind] += bytes;
  if (algo >= 0 && algo < ucclNumAlgos) c->counters.algoHist[algo]++;
}

ucclResult_t commPollDeviceStatus(Comm* c) {
  if (!c->hostFlags) return ucclSuccess;
  const uint32_t code = __atomic_load_n(&c->hostFlags[8], __ATOMIC_ACQUIRE);
  if (code == DEV_OK) return ucclSuccess;
  static const char* names[] = {"ok", "rank barrier", "low-latency receive", "point-to-point FIFO",
                                "network FIFO", "RMA signal", "fused GEMM flag", "MoE counter"};
  const char* what = code < 8 ? names[code] : (code == DEV_ABORTED ? "abort" : "unknown");
  commSetError(c, "device-side wait expired (%s): rank %u peer %u step %u block %u", what, c->hostFlags[9],
               c->hostFlags[10], c->hostFlags[11], c->hostFlags[12]);
  {
    std::lock_guard<std::mutex> lk(c->ctrMu);
    c->counters.waitTimeouts++;
  }
  commSetAsyncError(c, ucclRemoteError);
  // leave the abort word raised so that every later kernel returns at its first wait
  __atomic_store_n(&c->hostFlags[0], 1u, __ATOMIC_RELEASE);
  __atomic_store_n(&c->hostFlags[8], 0u, __ATOMIC_RELEASE);
  return ucclRemoteError;
}

void traceDump(Comm* c) {
  if (c->trace.empty()) return;
  FILE* f = nullptr;
  if (!c->cfg.traceFile.empty()) {
    char path[600];
    snprintf(path, sizeof(path), "%s.%d", c->cfg.traceFile.c_str(), c->rank);
    f = fopen(path, "w");
  }
  for (TraceEvent& t : c->trace) {
    float ms = 0.f;
    if (f && t.start && t.stop && cudaEventElapsedTime(&ms, t.start, t.stop) == cudaSuccess)
      fprintf(f, "{\"op\": \"%s\", \"bytes\": %zu, \"algo\": \"%s\", \"us\": %.2f}\n", t.name, t.bytes,
              algoName(static_cast<ucclAlgo_t>(t.algo)), ms * 1e3f);
    if (t.start) cudaEventDestroy(t.start);
    if (t.stop) cudaEventDestroy(t.stop);
  }
  (void)cudaGetLastError();
  if (f) fclose(f);
  c->trace.clear();
}

namespace {

ucclResult_t setupCuda(Comm* c) {
  // abort + status words: mapped host memory that kernels can read and write
  void* p = nullptr;
  if (cudaHostAlloc(&p, 64 * sizeof(uint32_t), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    commSetError(c, "cudaHostAlloc failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  memset(p, 0, 64 * sizeof(uint32_t));
  c->hostFlags = static_cast<uint32_t*>(p);
  void* d = nullptr;
  cudaHostGetDevicePointer(&d, p, 0);
  c->hostFlagsDev = static_cast<uint32_t*>(d);

  if (cudaMalloc(&p, (kMaxBlocks + kLLBlocks + 64) * sizeof(uint32_t)) != cudaSuccess) {
    commSetError(c, "cudaMalloc failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  cudaMemset(p, 0, (kMaxBlocks + kLLBlocks + 64) * sizeof(uint32_t));
  c->epochsDev = static_cast<uint32_t*>(p);

  DevComm& dc = c->dev;
  dc.rank = c->localRank;
  dc.nranks = c->localRanks;
  dc.epochs = c->epochsDev;
  dc.llEpochs = c->epochsDev + kMaxBlocks;
  dc.abortFlag = c->hostFlagsDev;
  dc.status = c->hostFlagsDev + 8;
  dc.timeoutNs = c->cfg.waitTimeoutMs * 1000000ull;
  return ucclSuccess;
}

ucclResult_t setupArena(Comm* c) {
  ucclResult_t r = c->heap.init(&c->bootstrap, c->localGlobalRanks, c->localRank, c->cudaDev, c->cfg);
  if (r != ucclSuccess) return r;
  const size_t p2pBytes = static_cast<size_t>(c->localRanks) * kP2pSlots * kP2pSlotBytes;
  const size_t staging = (c->cfg.stagingBytes + 4095) & ~size_t(4095);
  const size_t total = kArenaP2pDataOff + p2pBytes + staging;
  r = c->heap.alloc(total, &c->arena);
  if (r != ucclSuccess) {
    commSetError(c, "cannot create the symmetric arena (%zu bytes)", total);
    return r;
  }
  // zero the control part (flags, counters, LL lines); staging needs no clearing
  if (cudaMemset(c->arena->local, 0, kArenaP2pDataOff) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    commSetError(c, "arena memset failed: %s", cudaGetErrorString(cudaGetLastError()));
    return ucclSystemError;
  }
  for (int i = 0; i < c->localRanks; ++i) c->dev.arena[i] = c->arena->peer[i];
  c->dev.arenaMc = c->arena->mc;
  c->p2pReady = true;
  return c->bootstrap.barrier();  // nobody touches a peer's flags before they are cleared
}

void buildChannels(Comm* c) {
  // ring order: nodes in order, inside a node the topology's socket-grouped order
  std::vector<int> order;
  if (c->nNodes == 1 && !c->topo.gpus.empty() && static_cast<int>(c->topo.gpus.size()) == c->localRanks) {
    for (int li : topoRingOrder(c->topo)) order.push_back(c->localGlobalRanks[li]);
  } else {
    std::vector<std::pair<int, int>> keyed;
    for (const PeerInfo& p : c->peers) keyed.push_back({p.node * UCCL_MAX_RANKS + p.localRank, p.rank});
    std::sort(keyed.begin(), keyed.end());
    for (auto& kv : keyed) order.push_back(kv.second);
  }
  const int n = c->nRanks;
  int pos = 0;
  for (int i = 0; i < n; ++i)
    if (order[i] == c->rank) pos = i;
  c->channels.assign(c->nChannels, Channel());
  for (int ch = 0; ch < c->nChannels; ++ch) {
    Channel& k = c->channels[ch];
    k.id = ch;
    k.index = pos;
    k.prev = order[(pos + n - 1) % n];
    k.next = order[(pos + 1) % n];
    k.userRanks.resize(n);
    for (int i = 0; i < n; ++i) k.userRanks[i] = order[(pos + i) % n];
  }
}

// The algorithm and CTA count per message size come from a table measured on this kind of machine
// when one ships with the library: the directory "tuning" beside libuccl.so (or
// ../share/uccl/tuning for an installed copy, or UCCL_TUNE_DIR) is searched for a table whose GPU
// name, rank count and NVLS flag match this communicator.  UCCL_TUNE_FILE, when set, wins;
// UCCL_TUNE_AUTO=0 keeps the built-in priors.  Replaces the fixed thresholds of the reference
// (src/enqueue.cc:139-148, src/topo/topo_ring.cc:151-175).
void autoLoadTuning(Comm* c) {
  if (!c->cfg.tuneFile.empty() || c->backend != BACKEND_CUDA || !c->p2pReady || c->useNet || c->nRanks < 2) return;
  if (const char* e = getenv("UCCL_TUNE_AUTO")) {
    if (*e && atoi(e) == 0) return;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, c->cudaDev) != cudaSuccess) {
    (void)cudaGetLastError();
    return;
  }
  std::vector<std::string> dirs;
  if (const char* e = getenv("UCCL_TUNE_DIR")) {
    if (*e) dirs.push_back(e);
  }
  Dl_info info;
  if (dladdr(reinterpret_cast<const void*>(&autoLoadTuning), &info) && info.dli_fname) {
    std::string lib = info.dli_fname;
    const size_t slash = lib.rfind('/');
    const std::string dir = slash == std::string::npos ? "." : lib.substr(0, slash);
    dirs.push_back(dir + "/tuning");
    dirs.push_back(dir + "/../share/uccl/tuning");
  }
  for (const std::string& d : dirs) {
    std::string chosen;
    if (c->tuner.loadMatching(d, prop.name, c->nRanks, c->heap.nvls(), &chosen)) {
      c->tuneTable = chosen;
      UCCL_LOG(INFO, "tuning table %s", chosen.c_str());
      return;
    }
  }
}

ucclResult_t initRank(Comm* c, const ucclUniqueId& id) {
  ucclResult_t r;
  c->cfg = loadConfig();
  c->forcedAlgo = c->cfg.algo;
  c->forcedProto = c->cfg.proto;

  // backend
  int ndev = 0;
  if (c->cfg.backend != BACKEND_CPU) {
    if (cudaGetDeviceCount(&ndev) != cudaSuccess) {
      (void)cudaGetLastError();
      ndev = 0;
    }
  }
  if (c->cfg.backend == BACKEND_CUDA && ndev == 0) {
    commSetError(c, "UCCL_BACKEND=cuda but no CUDA device is visible");
    return ucclSystemError;
  }
  c->backend = ndev > 0 ? BACKEND_CUDA : BACKEND_CPU;
  if (c->backend == BACKEND_CUDA) {
    if (cudaGetDevice(&c->cudaDev) != cudaSuccess) {
      commSetError(c, "cudaGetDevice failed: %s", cudaGetErrorString(cudaGetLastError()));
      return ucclSystemError;
    }
    cudaFree(0);  // make sure the primary context exists before any driver call
  }

  UCCL_LOG(TRACE, "init: backend %s dev %d, starting bootstrap", c->backend == BACKEND_CUDA ? "cuda" : "cpu", c->cudaDev);
  r = c->bootstrap.init(id, c->rank, c->nRanks, c->cfg, &c->abortFlag);
  UCCL_LOG(TRACE, "init: bootstrap done (%d)", (int)r);
  if (r != ucclSuccess) {
    commSetError(c, "bootstrap failed: %s", c->bootstrap.lastError().c_str());
    return r;
  }

  // peer table
  c->peers.assign(c->nRanks, PeerInfo());
  PeerInfo& me = c->peers[c->rank];
  memset(&me, 0, sizeof(me));
  me.rank = c->rank;
  me.cudaDev = c->cudaDev;
  me.hostHash = getHostHash();
  me.pidHash = getPidHash();
  me.backend = c->backend;
  if (c->backend == BACKEND_CUDA) {
    char bus[32] = {0};
    if (cudaDeviceGetPCIBusId(bus, sizeof(bus), c->cudaDev) == cudaSuccess) me.busId = parseBusId(bus);
  }
  if ((r = c->bootstrap.allGather(c->peers.data(), sizeof(PeerInfo))) != ucclSuccess) {
    commSetError(c, "peer-info exchange failed: %s", c->bootstrap.lastError().c_str());
    return r;
  }
  std::vector<uint64_t> hosts;
  for (const PeerInfo& p : c->peers)
    if (std::find(hosts.begin(), hosts.end(), p.hostHash) == hosts.end()) hosts.push_back(p.hostHash);
  c->nNodes = static_cast<int>(hosts.size());
  c->localGlobalRanks.clear();
  for (PeerInfo& p : c->peers) {
    p.node = static_cast<int>(std::find(hosts.begin(), hosts.end(), p.hostHash) - hosts.begin());
    if (p.backend != c->backend) {
      commSetError(c, "rank %d runs the %s backend but rank %d does not", c->rank,
                   c->backend == BACKEND_CUDA ? "CUDA" : "CPU", p.rank);
      return ucclInvalidUsage;
    }
  }
  c->node = c->peers[c->rank].node;
  for (PeerInfo& p : c->peers) {
    if (p.node == c->node) {
      p.localRank = static_cast<int>(c->localGlobalRanks.size());
      c->localGlobalRanks.push_back(p.rank);
    }
  }
  // localRank of peers on other nodes: position among their own node's ranks
  {
    std::vector<int> counter(c->nNodes, 0);
    for (PeerInfo& p : c->peers) p.localRank = counter[p.node]++;
  }
  c->localRank = c->peers[c->rank].localRank;
  c->localRanks = static_cast<int>(c->localGlobalRanks.size());

  UCCL_LOG(TRACE, "init: peers exchanged, nodes=%d localRanks=%d", c->nNodes, c->localRanks);
  // topology + tuner priors
  bool p2pCapable = false;
  if (c->backend == BACKEND_CUDA) {
    std::vector<int> devs;
    for (int gr : c->localGlobalRanks) devs.push_back(c->peers[gr].cudaDev);
    if (topoDetect(&c->topo, devs) == ucclSuccess)
      p2pCapable = c->topo.allP2p && c->localRanks <= UCCL_MAX_LOCAL_RANKS;
    // two ranks on one device cannot run kernels that wait on each other
    std::set<int> distinct(devs.begin(), devs.end());
    if (static_cast<int>(distinct.size()) != c->localRanks) p2pCapable = false;
  }
  if (!c->cfg.tuneFile.empty()) {
    std::string why;
    if (!c->tuner.loadFile(c->cfg.tuneFile, &why))
      UCCL_LOG(WARN, "UCCL_TUNE_FILE=%s ignored: %s", c->cfg.tuneFile.c_str(), why.c_str());
  }

  // every rank must reach the same verdict on P2P
  if (c->nRanks > 1) {
    std::vector<uint8_t> v(c->nRanks, 0);
    v[c->rank] = p2pCapable ? 1 : 0;
    if ((r = c->bootstrap.allGather(v.data(), 1)) != ucclSuccess) return r;
    for (uint8_t b : v)
      if (!b) p2pCapable = false;
  }
  const bool multiNode = c->nNodes > 1;
  c->useNet = c->nRanks > 1 && (multiNode || c->cfg.forceNet || c->backend == BACKEND_CPU || !p2pCapable);

  UCCL_LOG(TRACE, "init: p2pCapable=%d useNet=%d", (int)p2pCapable, (int)c->useNet);
  if (c->backend == BACKEND_CUDA) {
    if ((r = setupCuda(c)) != ucclSuccess) return r;
    UCCL_LOG(TRACE, "init: device state ready");
    if (!multiNode && p2pCapable && c->nRanks >= 1) {
      if ((r = setupArena(c)) != ucclSuccess) {
        if (c->nRanks == 1) return r;
        UCCL_LOG(WARN, "symmetric arena unavailable; collectives will use the network path");
        c->p2pReady = false;
        c->useNet = c->nRanks > 1;
      }
    }
  }

  // channels
  if (c->cfg.nChannels > 0) c->nChannels = std::min(c->cfg.nChannels, UCCL_MAX_CHANNELS);
  else if (c->backend == BACKEND_CUDA && !c->topo.gpus.empty()) c->nChannels = std::min(topoTune(c->topo, 1u << 20).nChannels, UCCL_MAX_CHANNELS);
  else c->nChannels = c->nRanks <= 2 ? 2 : 4;
  if (c->useNet) c->nChannels = std::min(c->nChannels, 4);
  buildChannels(c);

  // network path
  if (c->useNet) {
    c->net = autoLoadNetPlugin(c->cfg.netPlugin);
    if ((r = c->net->init(&c->netContext)) != ucclSuccess) {
      commSetError(c, "network plugin %s failed to initialise", c->net->name);
      return r;
    }
    int nd = 0;
    c->net->devices(&nd);
    if (nd > 0) c->net->getProperties(0, &c->netProps);
    if ((r = netSetupRings(c)) != ucclSuccess) return r;
    if ((r = proxyStart(c)) != ucclSuccess) return r;
  }
  autoLoadTuning(c);
  logSetRank(c->rank);
  UCCL_LOG(INFO, "communicator ready: rank %d/%d node %d/%d backend %s p2p %d nvls %d net %s channels %d", c->rank,
           c->nRanks, c->node, c->nNodes, c->backend == BACKEND_CUDA ? "cuda" : "cpu", (int)c->p2pReady,
           (int)c->heap.nvls(), c->useNet ? c->net->name : "-", c->nChannels);
  return c->bootstrap.barrier();
}

void destroyComm(Comm* c) {
  proxyStop(c);
  if (c->backend == BACKEND_CUDA && c->cudaDev >= 0) cudaSetDevice(c->cudaDev);
  netTeardown(c);
  if (c->net && c->netContext) c->net->finalize(c->netContext);
  c->net = nullptr;
  c->netContext = nullptr;
  rmaDestroyAll(c);
  if (c->backend == BACKEND_CUDA) {
    cudaDeviceSynchronize();
    // peers may still be reading our arena in their last kernel: wait for everybody
    if (!c->abortFlag.load() && c->asyncError.load() == ucclSuccess) c->bootstrap.barrier();
    c->heap.releaseAll();
    for (int i = 0; i < UCCL_MAX_LOCAL_RANKS; ++i) {
      if (c->ceStream[i]) cudaStreamDestroy(c->ceStream[i]);
      if (c->ceEvent[i]) cudaEventDestroy(c->ceEvent[i]);
    }
    if (c->ceStart) cudaEventDestroy(c->ceStart);
    if (c->onesDev) cudaFree(c->onesDev);
    if (c->netScratch) cudaFree(c->netScratch);
    if (c->epochsDev) cudaFree(c->epochsDev);
    if (c->hostFlags) cudaFreeHost(c->hostFlags);
    traceDump(c);
  }
  c->bootstrap.close();
  c->magic = 0;
  delete c;
}

}  // namespace
}  // namespace uccl

using namespace uccl;

extern "C" ucclResult_t ucclGetUniqueId(ucclUniqueId* uniqueId) {
  if (!uniqueId) return ucclInvalidArgument;
  logBanner();
  Config cfg = loadConfig();
  return bootstrapCreateRoot(uniqueId, cfg);
}

extern "C" ucclResult_t ucclCommInitRank(ucclComm_t* comm, int nranks, ucclUniqueId commId, int rank) {
  logBanner();
  if (!comm) return ucclInvalidArgument;
  *comm = nullptr;
  if (nranks < 1 || nranks > UCCL_MAX_RANKS || rank < 0 || rank >= nranks) return ucclInvalidArgument;
  Comm* c = new Comm();
  c->rank = rank;
  c->nRanks = nranks;
  ucclResult_t r = initRank(c, commId);
  if (r != ucclSuccess) {
    UCCL_LOG(ERROR, "ucclCommInitRank(rank %d of %d) failed: %s (%s)", rank, nranks, ucclGetErrorString(r),
             c->lastError);
    c->abortFlag.store(1);
    destroyComm(c);
    return r;
  }
  *comm = reinterpret_cast<ucclComm_t>(c);
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommInitAll(ucclComm_t* comm, int ndev, const int* devlist) {
  if (!comm || ndev < 1 || ndev > UCCL_MAX_RANKS) return ucclInvalidArgument;
  int visible = 0;
  if (cudaGetDeviceCount(&visible) != cudaSuccess) {
    (void)cudaGetLastError();
    visible = 0;
  }
  ucclUniqueId id;
  ucclResult_t r = ucclGetUniqueId(&id);
  if (r != ucclSuccess) return r;
  std::vector<ucclResult_t> res(ndev, ucclSuccess);
  std::vector<std::thread> th;
  int prevDev = 0;
  if (visible > 0) cudaGetDevice(&prevDev);
  for (int i = 0; i < ndev; ++i) {
    const int dev = devlist ? devlist[i] : i;
    if (visible > 0 && (dev < 0 || dev >= visible)) return ucclInvalidArgument;
    th.emplace_back([&, i, dev] {
      if (visible > 0) cudaSetDevice(dev);
      res[i] = ucclCommInitRank(&comm[i], ndev, id, i);
    });
  }
  for (auto& t : th) t.join();
  if (visible > 0) cudaSetDevice(prevDev);
  for (int i = 0; i < ndev; ++i)
    if (res[i] != ucclSuccess) {
      for (int j = 0; j < ndev; ++j)
        if (res[j] == ucclSuccess && comm[j]) {
          ucclCommAbort(comm[j]);
          comm[j] = nullptr;
        }
      return res[i];
    }
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommFinalize(ucclComm_t comm) {
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  if (c->backend == BACKEND_CUDA) {
    cudaSetDevice(c->cudaDev);
    // bounded: kernels themselves give up after the wait budget, so this returns
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
      commSetError(c, "device synchronisation failed: %s", cudaGetErrorString(e));
      return ucclSystemError;
    }
    ucclResult_t r = commPollDeviceStatus(c);
    if (r != ucclSuccess) return r;
  }
  c->finalized = true;
  return static_cast<ucclResult_t>(c->asyncError.load());
}

extern "C" ucclResult_t ucclCommDestroy(ucclComm_t comm) {
  Comm* c = toComm(comm);
  if (!c) return ucclSuccess;
  if (!commValid(c)) return ucclInvalidArgument;
  destroyComm(c);
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommAbort(ucclComm_t comm) {
  Comm* c = toComm(comm);
  if (!c) return ucclSuccess;
  if (!commValid(c)) return ucclInvalidArgument;
  c->abortFlag.store(1);
  if (c->hostFlags) __atomic_store_n(&c->hostFlags[0], 1u, __ATOMIC_RELEASE);  // kernels poll this word
  destroyComm(c);
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommCount(const ucclComm_t comm, int* count) {
  const Comm* c = reinterpret_cast<const Comm*>(comm);
  if (!commValid(c) || !count) return ucclInvalidArgument;
  *count = c->nRanks;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommUserRank(const ucclComm_t comm, int* rank) {
  const Comm* c = reinterpret_cast<const Comm*>(comm);
  if (!commValid(c) || !rank) return ucclInvalidArgument;
  *rank = c->rank;
  return ucclSuccess;
}

extern "C" const char* ucclGetLastError(ucclComm_t comm) {
  Comm* c = toComm(comm);
  if (!commValid(c)) return "invalid communicator";
  return c->lastError;
}

extern "C" ucclResult_t ucclCommGetAsyncError(ucclComm_t comm, ucclResult_t* asyncError) {
  Comm* c = toComm(comm);
  if (!commValid(c) || !asyncError) return ucclInvalidArgument;
  if (c->backend == BACKEND_CUDA) commPollDeviceStatus(c);
  *asyncError = static_cast<ucclResult_t>(c->asyncError.load());
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommGetInfo(ucclComm_t comm, ucclCommInfo_t* info) {
  Comm* c = toComm(comm);
  if (!commValid(c) || !info) return ucclInvalidArgument;
  memset(info, 0, sizeof(*info));
  info->rank = c->rank;
  info->nranks = c->nRanks;
  info->nnodes = c->nNodes;
  info->localRank = c->localRank;
  info->localRanks = c->localRanks;
  info->cudaDevice = c->backend == BACKEND_CUDA ? c->cudaDev : -1;
  info->nChannels = c->nChannels;
  info->nvlsSupported = c->p2pReady && c->arena && c->arena->mc ? 1 : 0;
  info->p2pMode = c->p2pReady ? c->heap.mode() : 0;
  info->netActive = c->useNet ? 1 : 0;
  if (c->net) snprintf(info->netName, sizeof(info->netName), "%s", c->net->name);
  info->stagingBytes = c->p2pReady ? c->cfg.stagingBytes : 0;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommGetCounters(ucclComm_t comm, ucclCounters_t* counters) {
  Comm* c = toComm(comm);
  if (!commValid(c) || !counters) return ucclInvalidArgument;
  std::lock_guard<std::mutex> lk(c->ctrMu);
  *counters = c->counters;
  counters->proxyPosts = c->proxy.posts.load();
  counters->proxyCompletions = c->proxy.completions.load();
  counters->proxyHeartbeat = c->proxy.heartbeat.load();
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommLoadTuning(ucclComm_t comm, const char* jsonPath) {
  Comm* c = toComm(comm);
  if (!commValid(c) || !jsonPath) return ucclInvalidArgument;
  std::string why;
  if (!c->tuner.loadFile(jsonPath, &why)) {
    commSetError(c, "tuning table %s rejected: %s", jsonPath, why.c_str());
    return ucclInvalidArgument;
  }
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommSetAlgo(ucclComm_t comm, ucclAlgo_t algo, ucclProto_t proto) {
  Comm* c = toComm(comm);
  if (!commValid(c) || algo < 0 || algo >= ucclNumAlgos || proto < 0 || proto >= ucclNumProtos)
    return ucclInvalidArgument;
  c->forcedAlgo = algo;
  c->forcedProto = proto;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommSetFusedOptions(ucclComm_t comm, int agMode, int commCtas, int ceChunks) {
  Comm* c = toComm(comm);
  if (!commValid(c)) return ucclInvalidArgument;
  if (agMode < 0 || agMode > 3 || commCtas < 0 || commCtas > 64 || ceChunks < 0 || ceChunks > 64) return ucclInvalidArgument;
  c->fusedAgMode = agMode;
  c->fusedCommCtas = commCtas;
  c->fusedCeChunks = ceChunks;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommSetFusedRsReducers(ucclComm_t comm, int reducerCtas) {
  Comm* c = toComm(comm);
  if (!commValid(c) || reducerCtas < 0 || reducerCtas > 64) return ucclInvalidArgument;
  c->fusedRsReducers = reducerCtas;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommSetFusedNormRows(ucclComm_t comm, int rows) {
  Comm* c = toComm(comm);
  if (!commValid(c) || rows < -1 || rows > 4) return ucclInvalidArgument;
  c->fusedNormRows = rows;
  return ucclSuccess;
}

extern "C" ucclResult_t ucclCommSetBlocks(ucclComm_t comm, int blocks) {
  Comm* c = toComm(comm);
  if (!commValid(c) || blocks < 0 || blocks > kMaxBlocks) return ucclInvalidArgument;
  c->forcedBlocks = blocks;
  return ucclSuccess;
}

// A unique id derived from a rendezvous address that every rank already knows (for launchers that
// hand out MASTER_ADDR / MASTER_PORT): all ranks compute the same id, one of them serves it.
extern "C" ucclResult_t ucclUniqueIdFromAddress(const char* ip, int port, uint64_t seed, ucclUniqueId* id) {
  return uccl::bootstrapIdFromAddress(ip, port, seed, id);
}
extern "C" ucclResult_t ucclServeUniqueId(const ucclUniqueId* id) {
  if (!id) return ucclInvalidArgument;
  return uccl::bootstrapServeId(*id, uccl::loadConfig());
}
