#include "config.h"

#include <ctype.h>
#include <stdlib.h>
#include <string.h>
#include <stdint.h>
#include <strings.h>
#include <time.h>

#include "log.h"

namespace uccl {

bool parseAlgo(const char* s, ucclAlgo_t* out) {
  if (!s || !*s) return false;
  struct { const char* n; ucclAlgo_t a; } tab[] = {
      {"auto", ucclAlgoAuto},       {"ring", ucclAlgoRing},         {"one_shot", ucclAlgoOneShot},
      {"oneshot", ucclAlgoOneShot}, {"two_shot", ucclAlgoTwoShot},  {"twoshot", ucclAlgoTwoShot},
      {"symmetric", ucclAlgoTwoShot}, {"nvls", ucclAlgoNvls},       {"copy_engine", ucclAlgoCopyEngine},
      {"ce", ucclAlgoCopyEngine},   {"net", ucclAlgoNet}};
  for (auto& t : tab)
    if (!strcasecmp(s, t.n)) { *out = t.a; return true; }
  return false;
}

bool parseProto(const char* s, ucclProto_t* out) {
  if (!s || !*s) return false;
  struct { const char* n; ucclProto_t p; } tab[] = {
      {"auto", ucclProtoAuto}, {"simple", ucclProtoSimple}, {"ll", ucclProtoLL}, {"ll128", ucclProtoLL128}};
  for (auto& t : tab)
    if (!strcasecmp(s, t.n)) { *out = t.p; return true; }
  return false;
}

const char* algoName(ucclAlgo_t a) {
  switch (a) {
    case ucclAlgoAuto: return "auto";
    case ucclAlgoRing: return "ring";
    case ucclAlgoOneShot: return "one_shot";
    case ucclAlgoTwoShot: return "two_shot";
    case ucclAlgoNvls: return "nvls";
    case ucclAlgoCopyEngine: return "copy_engine";
    case ucclAlgoNet: return "net";
    default: return "?";
  }
}
const char* protoName(ucclProto_t p) {
  switch (p) {
    case ucclProtoAuto: return "auto";
    case ucclProtoSimple: return "simple";
    case ucclProtoLL: return "ll";
    case ucclProtoLL128: return "ll128";
    default: return "?";
  }
}

size_t parseSize(const char* s, size_t dflt) {
  if (!s || !*s) return dflt;
  char* end = nullptr;
  double v = strtod(s, &end);
  if (end == s || v < 0) return dflt;
  while (*end && isspace((unsigned char)*end)) ++end;
  switch (tolower((unsigned char)*end)) {
    case 'k': v *= 1024.0; break;
    case 'm': v *= 1024.0 * 1024.0; break;
    case 'g': v *= 1024.0 * 1024.0 * 1024.0; break;
    default: break;
  }
  return static_cast<size_t>(v);
}

static long envLong(const char* name, long dflt) {
  const char* s = getenv(name);
  if (!s || !*s) return dflt;
  char* end = nullptr;
  long v = strtol(s, &end, 10);
  return end == s ? dflt : v;
}

Config loadConfig() {
  Config c;
  const char* s;
  if ((s = getenv("UCCL_ALGO")) && *s && !parseAlgo(s, &c.algo))
    UCCL_LOG(WARN, "UCCL_ALGO=%s not recognised; using the tuner", s);
  if ((s = getenv("UCCL_PROTO")) && *s && !parseProto(s, &c.proto))
    UCCL_LOG(WARN, "UCCL_PROTO=%s not recognised; using the tuner", s);
  c.nChannels = (int)envLong("UCCL_NCHANNELS", 0);
  if (c.nChannels < 0) c.nChannels = 0;
  c.maxCtas = (int)envLong("UCCL_MAX_CTAS", envLong("UCCL_EU_COUNT", 0));
  if ((s = getenv("UCCL_EXEC_MODE")) && *s) {
    if (!strcasecmp(s, "copy_engine") || !strcasecmp(s, "ce")) c.execMode = EXEC_COPY_ENGINE;
    else if (!strcasecmp(s, "hybrid")) c.execMode = EXEC_HYBRID;
  }
  if ((s = getenv("UCCL_NET_PLUGIN")) && *s) c.netPlugin = s;
  c.forceNet = envLong("UCCL_FORCE_NET", 0) == 1;
  if ((s = getenv("UCCL_TUNE_FILE")) && *s) c.tuneFile = s;
  {
    // every device-side wait stays bounded: 1 ms .. 10 min, whatever the variable says
    long ms = envLong("UCCL_WAIT_TIMEOUT_MS", 10000);
    if (ms < 1 || ms > 600000) {
      const long clamped = ms < 1 ? 1 : 600000;
      UCCL_LOG(WARN, "UCCL_WAIT_TIMEOUT_MS=%ld is outside [1, 600000]; using %ld", ms, clamped);
      ms = clamped;
    }
    c.waitTimeoutMs = (uint64_t)ms;
  }
  c.nvls = (int)envLong("UCCL_NVLS", -1);
  if ((s = getenv("UCCL_BOOTSTRAP_IFNAME")) && *s) c.bootstrapIf = s;
  c.bootstrapPort = (int)envLong("UCCL_BOOTSTRAP_PORT", 0);
  c.bootstrapTimeoutMs = (uint64_t)envLong("UCCL_BOOTSTRAP_TIMEOUT_MS", 60000);
  c.stagingBytes = parseSize(getenv("UCCL_STAGING_BYTES"), 64ull << 20);
  if ((s = getenv("UCCL_BACKEND")) && *s) {
    if (!strcasecmp(s, "cpu") || !strcasecmp(s, "host")) c.backend = BACKEND_CPU;
    else if (!strcasecmp(s, "cuda") || !strcasecmp(s, "gpu")) c.backend = BACKEND_CUDA;
  }
  if ((s = getenv("UCCL_P2P")) && *s) {
    if (!strcasecmp(s, "ipc")) c.p2pMode = 1;
    else if (!strcasecmp(s, "vmm")) c.p2pMode = 2;
  }
  if ((s = getenv("UCCL_TRACE_FILE")) && *s) c.traceFile = s;
  c.netChunkBytes = parseSize(getenv("UCCL_NET_CHUNK_BYTES"), 512u << 10);
  if (c.netChunkBytes < 4096) c.netChunkBytes = 4096;
  c.jitterUs = (int)envLong("UCCL_JITTER_US", 0);
  if (c.jitterUs < 0) c.jitterUs = 0;
  c.canary = envLong("UCCL_CANARY", 0) != 0;
  c.fusedCeChunks = (int)envLong("UCCL_FUSED_CE_CHUNKS", 0);
  if (c.fusedCeChunks < 0) c.fusedCeChunks = 0;
  return c;
}

void jitterPause(int maxUs) {
  if (maxUs <= 0) return;
  static thread_local uint64_t state = 0x9e3779b97f4a7c15ull ^ reinterpret_cast<uintptr_t>(&state);
  state ^= state << 13;
  state ^= state >> 7;
  state ^= state << 17;
  const long us = static_cast<long>(state % static_cast<uint64_t>(maxUs + 1));
  if (us == 0) return;
  struct timespec ts = {0, us * 1000};
  nanosleep(&ts, nullptr);
}

}  // namespace uccl
