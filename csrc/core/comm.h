// The communicator: all per-rank state.  Counterpart of the reference's ucclComm
// (src/include/comm.h:55-101), with the fields that were declared but never initialised there
// (device, default queue, topology, symmetric context, hardware resources) actually owned and
// set up by init.cc.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../kernels/device_comm.h"
#include "../mem/symmem.h"
#include "../transport/net_conn.h"
#include "bootstrap.h"
#include "config.h"
#include "topo.h"
#include "tuner.h"
#include "uccl.h"
#include "uccl_net.h"

namespace uccl {

struct PeerInfo {
  int32_t rank;
  int32_t localRank;
  int32_t node;
  int32_t cudaDev;
  uint64_t hostHash;
  uint64_t pidHash;
  int64_t busId;
  int32_t backend;  // BackendKind actually in use
  int32_t pad;
};

struct Channel {
  int id = 0;
  int prev = 0, next = 0;              // ring neighbours (communicator ranks)
  std::vector<int> userRanks;          // ring order starting at this rank
  int index = 0;                       // position of this rank in the ring order
  NetConn send, recv;                  // to next / from prev (network path only)
  bool netReady = false;
};

struct ProxyState {
  std::thread thread;
  std::atomic<bool> stop{false};
  std::atomic<bool> running{false};
  std::atomic<uint64_t> heartbeat{0};
  std::atomic<uint64_t> posts{0};
  std::atomic<uint64_t> completions{0};
};

struct TraceEvent {
  const char* name;
  size_t bytes;
  int algo;
  cudaEvent_t start, stop;
};

struct Window;

struct Comm {
  uint32_t magic = 0x55434c43;  // validity stamp, cleared on destroy
  int rank = 0, nRanks = 1;
  int nNodes = 1, node = 0;
  int localRank = 0, localRanks = 1;
  std::vector<int> localGlobalRanks;  // communicator ranks sharing this host, ordered
  Config cfg;
  BackendKind backend = BACKEND_CPU;
  int cudaDev = -1;
  std::vector<PeerInfo> peers;
  Bootstrap bootstrap;

  // topology + tuning
  TopoSystem topo;
  Tuner tuner;
  void* netScratch = nullptr;  // device work copy of the network ring (reduce-scatter, reduce)
  size_t netScratchBytes = 0;
  std::string tuneTable;  // path of the shipped table that was loaded at creation, if any
  ucclAlgo_t forcedAlgo = ucclAlgoAuto;
  ucclProto_t forcedProto = ucclProtoAuto;
  int fusedAgMode = 0, fusedCommCtas = 0, fusedCeChunks = 0;  // ucclCommSetFusedOptions (0 = default)
  int forcedBlocks = 0;               // CTA count forced by ucclCommSetBlocks (0 = tuner)

  // NVLink domain
  SymHeap heap;
  SymSegment* arena = nullptr;
  bool p2pReady = false;
  DevComm dev{};                      // by-value kernel argument
  uint32_t* epochsDev = nullptr;      // device memory behind dev.epochs / dev.llEpochs
  uint32_t* hostFlags = nullptr;      // mapped host: [0] abort, [8..16) status
  uint32_t* hostFlagsDev = nullptr;
  uint32_t gemmEpoch = 0;             // arrival-flag epoch of the fused GEMM paths
  cudaStream_t ceStream[UCCL_MAX_LOCAL_RANKS] = {};
  cudaEvent_t ceEvent[UCCL_MAX_LOCAL_RANKS] = {};
  cudaEvent_t ceStart = nullptr;
  bool ceReady = false;
  int fusedRsReducers = 0;                  // ucclCommSetFusedRsReducers: CTAs that only sum
  int fusedNormRows = -1;                   // ucclCommSetFusedNormRows: rows per pass of the fused norm's all-reduce phase (-1 = default)
  void* onesDev = nullptr;            // 32-bit ones at the GEMM flag stride (source of copy-engine flag writes)

  // network path
  ucclNet_t* net = nullptr;
  void* netContext = nullptr;
  ucclNetProperties_t netProps{};
  bool useNet = false;                // collectives go through proxy + plugin
  int nChannels = 1;
  std::vector<Channel> channels;
  std::mutex netMu;                   // guards meshSend/meshRecv/allConns growth
  std::vector<std::unique_ptr<NetConn>> meshSend, meshRecv;  // indexed by peer
  std::vector<NetConn*> allConns;     // what the proxy iterates over
  ProxyState proxy;

  // RMA
  std::mutex winMu;
  std::vector<Window*> windows;

  // bookkeeping
  std::atomic<uint32_t> abortFlag{0};
  std::atomic<int> asyncError{ucclSuccess};
  std::mutex errMu;
  char lastError[256] = {0};
  ucclCounters_t counters{};
  std::mutex ctrMu;
  uint64_t opCount = 0;
  std::vector<TraceEvent> trace;
  bool finalized = false;
};

// ------------------------------------------------------------------ helpers (init.cc)
bool commValid(const Comm* c);
void commSetError(Comm* c, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void commSetAsyncError(Comm* c, ucclResult_t r);
// Reads the device status words; converts a recorded device-side failure into asyncError.
ucclResult_t commPollDeviceStatus(Comm* c);
inline Comm* toComm(ucclComm_t h) { return reinterpret_cast<Comm*>(h); }
uint64_t getHostHash();
uint64_t getPidHash();
size_t dataTypeSize(ucclDataType_t t);
void commCount(Comm* c, ucclCollKind_t kind, size_t bytes, ucclAlgo_t algo);

// proxy.cc
ucclResult_t proxyStart(Comm* c);
void proxyStop(Comm* c);
// Single progress pass over one connection (exposed for the self tests).
// Returns ucclSuccess, or the plugin's error code.
ucclResult_t proxyProgressConn(ucclNet_t* net, NetConn* conn, uint64_t* posts, uint64_t* completions);

}  // namespace uccl
