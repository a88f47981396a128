// Per-communicator configuration, parsed from the environment once at communicator creation.
// The reference reads each variable ad hoc where it is needed (UCCL_ALGO at
// src/enqueue.cc:105-117, UCCL_EXEC_MODE / UCCL_EU_COUNT at src/include/hw_resources.h:158-175,
// UCCL_NET_PLUGIN at src/plugin/net_ucx.cc:631-635, UCCL_FORCE_NET at src/transport.cc:42);
// here the same names are kept and gathered in one struct, plus the new knobs.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <string>

#include "uccl.h"

namespace uccl {

enum ExecMode : int { EXEC_SM_ONLY = 0, EXEC_COPY_ENGINE = 1, EXEC_HYBRID = 2 };
enum BackendKind : int { BACKEND_AUTO = 0, BACKEND_CUDA = 1, BACKEND_CPU = 2 };

struct Config {
  ucclAlgo_t algo = ucclAlgoAuto;        // UCCL_ALGO
  ucclProto_t proto = ucclProtoAuto;     // UCCL_PROTO
  int nChannels = 0;                     // UCCL_NCHANNELS (0 = tuner)
  int maxCtas = 0;                       // UCCL_MAX_CTAS (successor of UCCL_EU_COUNT)
  ExecMode execMode = EXEC_SM_ONLY;      // UCCL_EXEC_MODE = copy_engine|ce|hybrid
  std::string netPlugin;                 // UCCL_NET_PLUGIN
  bool forceNet = false;                 // UCCL_FORCE_NET=1
  std::string tuneFile;                  // UCCL_TUNE_FILE
  uint64_t waitTimeoutMs = 10000;        // UCCL_WAIT_TIMEOUT_MS (device-side waits)
  int nvls = -1;                         // UCCL_NVLS: -1 auto, 0 off, 1 required
  std::string bootstrapIf;               // UCCL_BOOTSTRAP_IFNAME
  int bootstrapPort = 0;                 // UCCL_BOOTSTRAP_PORT
  uint64_t bootstrapTimeoutMs = 60000;   // UCCL_BOOTSTRAP_TIMEOUT_MS
  size_t stagingBytes = 64ull << 20;     // UCCL_STAGING_BYTES
  BackendKind backend = BACKEND_AUTO;    // UCCL_BACKEND = cuda|cpu
  int p2pMode = 0;                       // UCCL_P2P = 0 auto, 1 cudaIpc, 2 vmm
  std::string traceFile;                 // UCCL_TRACE_FILE
  size_t netChunkBytes = 512u << 10;     // UCCL_NET_CHUNK_BYTES (bounce slot size)
  int jitterUs = 0;                      // UCCL_JITTER_US: random host-side pauses of up to this many microseconds (testing)
  bool canary = false;                   // UCCL_CANARY=1: guard words around every ucclMemAlloc buffer, verified by ucclMemCheck / ucclMemFree
  int fusedCeChunks = 0;                 // UCCL_FUSED_CE_CHUNKS: copies per peer of the copy-engine all-gather
};

Config loadConfig();

// Schedule perturbation for tests: sleeps a pseudo-random time in [0, maxUs] microseconds (per-thread
// generator); a no-op when maxUs <= 0.  Called between the steps of the proxy thread and of the
// host-driven transfer loop so that orderings which normally never occur get exercised.
void jitterPause(int maxUs);

// Parsers exposed for unit tests.
bool parseAlgo(const char* s, ucclAlgo_t* out);
bool parseProto(const char* s, ucclProto_t* out);
const char* algoName(ucclAlgo_t a);
const char* protoName(ucclProto_t p);
size_t parseSize(const char* s, size_t dflt);

}  // namespace uccl
