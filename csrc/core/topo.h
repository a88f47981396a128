// Topology model of one host's GPUs and the tuning defaults derived from it.
//
// The reference classifies Intel GPU pairs as PCIe-same-switch / PCIe-cross-switch / UPI / NET
// with nominal 64/32/40 GB/s figures (src/topo/topo.h:13-60, src/topo/topo_pci.cc:109-145), reads
// NUMA placement from sysfs (src/topo/topo_upi.cc:13-120), orders the ring so that it crosses the
// socket boundary exactly twice (src/topo/topo_ring.cc:21-98) and picks channel counts / chunk
// sizes from the GPU count and message size (src/topo/topo_ring.cc:140-207).  The same four jobs
// are done here for NVLink 5 / NVSwitch machines: link classes gain NVSWITCH and NVLINK, the
// information comes from the CUDA runtime and sysfs, and the tuning output feeds the measured
// tuner as its prior.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "uccl.h"

namespace uccl {

enum LinkType : int {
  LINK_SELF = 0,
  LINK_NVSWITCH = 1,     // NVLink through NVSwitch: uniform bandwidth to every peer
  LINK_NVLINK = 2,       // direct NVLink bricks between two GPUs
  LINK_PCIE_SWITCH = 3,  // same PCIe switch
  LINK_PCIE_HOST = 4,    // different switches, same socket (through the root complex)
  LINK_SYS = 5,          // different sockets (UPI / xGMI hop)
  LINK_NET = 6,
};

struct TopoGpu {
  int dev = -1;
  int rank = -1;
  std::string busId;    // "0000:1b:00.0"
  int64_t busIdNum = 0; // domain<<20 | bus<<12 | device<<4 | function
  int numaNode = -1;
  int socket = -1;
  int smCount = 0;
  int multicast = 0;
};

struct TopoLink {
  LinkType type = LINK_SELF;
  float bwGBs = 0.f;  // per direction
  float latUs = 0.f;
};

struct TopoTuning {
  int nChannels = 4;
  int nThreads = 512;
  size_t chunkBytes = 512u << 10;
  ucclAlgo_t algo = ucclAlgoRing;
  ucclProto_t proto = ucclProtoSimple;
  float bwGBs = 0.f;
  float latUs = 0.f;
};

struct TopoSystem {
  std::vector<TopoGpu> gpus;
  std::vector<TopoLink> links;  // gpus.size()^2, row-major [from][to]
  bool nvswitch = false;
  bool allP2p = false;
  const TopoLink& link(int a, int b) const { return links[a * gpus.size() + b]; }
};

// Raw facts about a GPU pair, as cudaDeviceGetP2PAttribute reports them.
struct P2pFacts {
  int access = 0;
  int nativeAtomics = 0;
  int perfRank = 0;
};

int64_t parseBusId(const std::string& s);
// NUMA node of a PCI device from sysfs (-1 if unknown); sysfsRoot lets tests point at a fixture.
int readNumaNode(const std::string& busId, const std::string& sysfsRoot = "/sys");
// Socket (physical package) that owns a NUMA node (-1 if unknown).
int numaToSocket(int numaNode, const std::string& sysfsRoot = "/sys");

// Pure classification used by detection and by the tests.
TopoLink classifyLink(const TopoGpu& a, const TopoGpu& b, const P2pFacts& f, bool nvswitch);
void topoBuildLinks(TopoSystem* sys, const std::vector<P2pFacts>& facts /* n*n */);

// Queries the CUDA runtime + sysfs for the listed devices (index i of devs = local rank i).
ucclResult_t topoDetect(TopoSystem* sys, const std::vector<int>& devs);

// Ring order: GPUs grouped by socket, sorted by bus id inside a socket, sockets concatenated.
std::vector<int> topoRingOrder(const TopoSystem& sys);
int topoSocketCrossings(const TopoSystem& sys, const std::vector<int>& order);

TopoTuning topoTune(const TopoSystem& sys, size_t bytes);
const char* linkTypeName(LinkType t);

}  // namespace uccl
