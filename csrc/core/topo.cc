#include "topo.h"

#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>

#include "cuda_driver.h"
#include "log.h"

namespace uccl {

const char* linkTypeName(LinkType t) {
  switch (t) {
    case LINK_SELF: return "SELF";
    case LINK_NVSWITCH: return "NVSWITCH";
    case LINK_NVLINK: return "NVLINK";
    case LINK_PCIE_SWITCH: return "PCIE_SWITCH";
    case LINK_PCIE_HOST: return "PCIE_HOST";
    case LINK_SYS: return "SYS";
    case LINK_NET: return "NET";
  }
  return "?";
}

int64_t parseBusId(const std::string& s) {
  unsigned dom = 0, bus = 0, dev = 0, fn = 0;
  if (sscanf(s.c_str(), "%x:%x:%x.%x", &dom, &bus, &dev, &fn) == 4)
    return (static_cast<int64_t>(dom) << 20) | (bus << 12) | (dev << 4) | fn;
  if (sscanf(s.c_str(), "%x:%x.%x", &bus, &dev, &fn) == 3) return (bus << 12) | (dev << 4) | fn;
  return -1;
}

static std::string lower(std::string s) {
  for (char& c : s) c = static_cast<char>(tolower(static_cast<unsigned char>(c)));
  return s;
}

// The sysfs readers use stdio on purpose: this shared object carries its own copy of the C++
// runtime, whose stream locale machinery is not set up when the object is loaded into a host
// process, so formatted iostream extraction is off limits in library code.
static bool readFirstLine(const std::string& path, char* buf, size_t len) {
  FILE* f = fopen(path.c_str(), "r");
  if (!f) return false;
  const bool ok = fgets(buf, static_cast<int>(len), f) != nullptr;
  fclose(f);
  return ok;
}

int readNumaNode(const std::string& busId, const std::string& sysfsRoot) {
  char buf[64];
  if (!readFirstLine(sysfsRoot + "/bus/pci/devices/" + lower(busId) + "/numa_node", buf, sizeof(buf))) return -1;
  char* end = nullptr;
  const long v = strtol(buf, &end, 10);
  return end == buf ? -1 : static_cast<int>(v);
}

int numaToSocket(int numaNode, const std::string& sysfsRoot) {
  if (numaNode < 0) return -1;
  char buf[256];
  char name[64];
  snprintf(name, sizeof(name), "%d", numaNode);
  if (!readFirstLine(sysfsRoot + "/devices/system/node/node" + name + "/cpulist", buf, sizeof(buf))) return -1;
  char* end = nullptr;
  const long cpu = strtol(buf, &end, 10);  // first CPU of the list ("0-31,64-95" -> 0)
  if (end == buf) return -1;
  snprintf(name, sizeof(name), "%ld", cpu);
  if (!readFirstLine(sysfsRoot + "/devices/system/cpu/cpu" + name + "/topology/physical_package_id", buf, sizeof(buf)))
    return -1;
  const long pkg = strtol(buf, &end, 10);
  return end == buf ? -1 : static_cast<int>(pkg);
}

TopoLink classifyLink(const TopoGpu& a, const TopoGpu& b, const P2pFacts& f, bool nvswitch) {
  TopoLink l;
  if (a.dev == b.dev && a.busIdNum == b.busIdNum) {
    l.type = LINK_SELF;
    l.bwGBs = 6500.f;
    l.latUs = 0.f;
    return l;
  }
  if (f.access && f.nativeAtomics) {
    // native atomics over the link is the signature of NVLink
    l.type = nvswitch ? LINK_NVSWITCH : LINK_NVLINK;
    l.bwGBs = 900.f;  // NVLink 5: 18 links x 50 GB/s per direction
    l.latUs = nvswitch ? 1.0f : 0.7f;
    return l;
  }
  const bool sameSocket = a.socket >= 0 && a.socket == b.socket;
  const bool knownSockets = a.socket >= 0 && b.socket >= 0;
  if (knownSockets && !sameSocket) {
    l.type = LINK_SYS;
    l.bwGBs = 40.f;
    l.latUs = 1.0f;
  } else if ((a.busIdNum >> 16) == (b.busIdNum >> 16)) {
    // same upper bus bits: behind one switch
    l.type = LINK_PCIE_SWITCH;
    l.bwGBs = 64.f;
    l.latUs = 0.1f;
  } else {
    l.type = LINK_PCIE_HOST;
    l.bwGBs = 32.f;
    l.latUs = 0.3f;
  }
  if (!f.access) {
    // no peer access at all: traffic bounces through host memory
    l.bwGBs *= 0.5f;
    l.latUs += 2.0f;
  }
  return l;
}

void topoBuildLinks(TopoSystem* sys, const std::vector<P2pFacts>& facts) {
  const size_t n = sys->gpus.size();
  sys->links.assign(n * n, TopoLink());
  bool all = true;
  for (size_t i = 0; i < n; ++i)
    for (size_t j = 0; j < n; ++j) {
      sys->links[i * n + j] = classifyLink(sys->gpus[i], sys->gpus[j], facts[i * n + j], sys->nvswitch);
      if (i != j && !facts[i * n + j].access) all = false;
    }
  sys->allP2p = all;
}

ucclResult_t topoDetect(TopoSystem* sys, const std::vector<int>& devs) {
  const size_t n = devs.size();
  sys->gpus.resize(n);
  int visible = 0;
  if (cudaGetDeviceCount(&visible) != cudaSuccess) {
    (void)cudaGetLastError();
    return ucclSystemError;
  }
  bool anyMc = false;
  for (size_t i = 0; i < n; ++i) {
    TopoGpu& g = sys->gpus[i];
    g.dev = devs[i];
    g.rank = static_cast<int>(i);
    if (g.dev < 0 || g.dev >= visible) continue;
    UCCL_LOG(TRACE, "topo: querying device %d", g.dev);
    char bus[32] = {0};
    if (cudaDeviceGetPCIBusId(bus, sizeof(bus), g.dev) == cudaSuccess) {
      UCCL_LOG(TRACE, "topo: bus id %s", bus);
      g.busId = bus;
      g.busIdNum = parseBusId(g.busId);
      UCCL_LOG(TRACE, "topo: bus num %lld", (long long)g.busIdNum);
      g.numaNode = readNumaNode(g.busId);
      UCCL_LOG(TRACE, "topo: numa %d", g.numaNode);
      g.socket = numaToSocket(g.numaNode);
    } else {
      (void)cudaGetLastError();
    }
    UCCL_LOG(TRACE, "topo: device %d bus %s numa %d socket %d", g.dev, g.busId.c_str(), g.numaNode, g.socket);
    cudaDeviceGetAttribute(&g.smCount, cudaDevAttrMultiProcessorCount, g.dev);
    UCCL_LOG(TRACE, "topo: device %d sms %d", g.dev, g.smCount);
    const DriverApi& d = driverApi();
    UCCL_LOG(TRACE, "topo: driver api ok=%d", (int)d.ok);
    if (d.ok) {
      CUdevice cd;
      int v = 0;
      if (d.deviceGet(&cd, g.dev) == CUDA_SUCCESS &&
          d.deviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) == CUDA_SUCCESS)
        g.multicast = v;
    }
    anyMc |= g.multicast != 0;
  }
  std::vector<P2pFacts> facts(n * n);
  for (size_t i = 0; i < n; ++i)
    for (size_t j = 0; j < n; ++j) {
      if (i == j) continue;
      const int a = devs[i], b = devs[j];
      if (a < 0 || b < 0 || a >= visible || b >= visible) continue;
      P2pFacts& f = facts[i * n + j];
      if (a == b) {  // several ranks on one device (test setups)
        f.access = 1;
        f.nativeAtomics = 1;
        continue;
      }
      UCCL_LOG(TRACE, "topo: p2p attributes %d -> %d", a, b);
      cudaDeviceGetP2PAttribute(&f.access, cudaDevP2PAttrAccessSupported, a, b);
      cudaDeviceGetP2PAttribute(&f.nativeAtomics, cudaDevP2PAttrNativeAtomicSupported, a, b);
      cudaDeviceGetP2PAttribute(&f.perfRank, cudaDevP2PAttrPerformanceRank, a, b);
      (void)cudaGetLastError();
    }
  // Multicast objects exist only behind an NVSwitch fabric.
  sys->nvswitch = anyMc;
  topoBuildLinks(sys, facts);
  if (logLevel() >= LOG_INFO) {
    for (size_t i = 0; i < n; ++i)
      UCCL_LOG(INFO, "topo: gpu %zu dev %d bus %s numa %d socket %d link-to-0 %s", i, sys->gpus[i].dev,
               sys->gpus[i].busId.c_str(), sys->gpus[i].numaNode, sys->gpus[i].socket,
               linkTypeName(sys->link(static_cast<int>(i), 0).type));
  }
  return ucclSuccess;
}

std::vector<int> topoRingOrder(const TopoSystem& sys) {
  std::vector<int> idx(sys.gpus.size());
  for (size_t i = 0; i < idx.size(); ++i) idx[i] = static_cast<int>(i);
  std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) {
    const TopoGpu& ga = sys.gpus[a];
    const TopoGpu& gb = sys.gpus[b];
    if (ga.socket != gb.socket) return ga.socket < gb.socket;
    return ga.busIdNum < gb.busIdNum;
  });
  return idx;
}

int topoSocketCrossings(const TopoSystem& sys, const std::vector<int>& order) {
  int crossings = 0;
  const size_t n = order.size();
  for (size_t i = 0; i < n; ++i) {
    const TopoGpu& a = sys.gpus[order[i]];
    const TopoGpu& b = sys.gpus[order[(i + 1) % n]];
    if (a.socket != b.socket) ++crossings;
  }
  return crossings;
}

TopoTuning topoTune(const TopoSystem& sys, size_t bytes) {
  TopoTuning t;
  const size_t n = sys.gpus.size();
  float minBw = 1e30f, maxLat = 0.f;
  bool sameSocket = true;
  for (size_t i = 0; i < n; ++i)
    for (size_t j = 0; j < n; ++j) {
      if (i == j) continue;
      const TopoLink& l = sys.links[i * n + j];
      minBw = std::min(minBw, l.bwGBs);
      maxLat = std::max(maxLat, l.latUs);
      if (sys.gpus[i].socket != sys.gpus[j].socket) sameSocket = false;
    }
  if (n <= 1) { minBw = 6500.f; maxLat = 0.f; }
  t.bwGBs = minBw;
  t.latUs = maxLat;
  t.nChannels = n <= 2 ? 2 : (n <= 4 ? 4 : 8);
  const bool fabric = sys.nvswitch || (n > 1 && sys.link(0, 1).type == LINK_NVLINK);
  if (fabric) {
    // full-bandwidth mesh: latency-optimal algorithms below the bandwidth knee
    t.nChannels *= 4;
    if (bytes < (64u << 10)) { t.algo = ucclAlgoOneShot; t.proto = ucclProtoLL; t.chunkBytes = 4u << 10; t.nThreads = 256; }
    else if (bytes <= (512u << 10)) { t.algo = ucclAlgoOneShot; t.proto = ucclProtoSimple; t.chunkBytes = 64u << 10; t.nThreads = 512; }
    else { t.algo = sys.nvswitch ? ucclAlgoNvls : ucclAlgoTwoShot; t.proto = ucclProtoSimple; t.chunkBytes = 512u << 10; t.nThreads = 512; }
    return t;
  }
  t.algo = ucclAlgoRing;
  if (bytes < (4u << 10)) { t.proto = ucclProtoLL128; t.chunkBytes = 4u << 10; t.nThreads = 256; }
  else if (bytes <= (512u << 10)) {
    if (sameSocket) { t.proto = ucclProtoLL128; t.chunkBytes = 64u << 10; t.nThreads = 256; }
    else { t.proto = ucclProtoSimple; t.chunkBytes = 64u << 10; t.nThreads = 512; }
  } else { t.proto = ucclProtoSimple; t.chunkBytes = 512u << 10; t.nThreads = 512; }
  return t;
}

}  // namespace uccl
