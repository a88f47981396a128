// Algorithm / protocol / CTA-count selection per (collective, message size).
//
// The reference hard-codes two thresholds (one-shot + LL128 below 4 KiB, ring + Simple above,
// src/enqueue.cc:121-181, and the LL128/Simple split at 512 KiB in src/topo/topo_ring.cc:151-175).
// Here the decision comes from a table of measured times per (collective, algorithm, protocol,
// size) written by the sweep benchmark as JSON: the tuner interpolates each feasible curve at the
// requested size and takes the fastest.  Without a table, built-in priors derived from the
// topology are used.  UCCL_ALGO / UCCL_PROTO / ucclCommSetAlgo override both.
#pragma once
#include <stddef.h>

#include <string>
#include <vector>

#include "uccl.h"

namespace uccl {

struct TunePoint {
  size_t bytes;
  float us;
  int blocks;
};

struct TuneCurve {
  ucclCollKind_t coll;
  ucclAlgo_t algo;
  ucclProto_t proto;
  std::vector<TunePoint> pts;  // sorted by bytes
};

struct TuneChoice {
  ucclAlgo_t algo = ucclAlgoTwoShot;
  ucclProto_t proto = ucclProtoSimple;
  int blocks = 8;
  bool fromTable = false;
};

struct TuneQuery {
  ucclCollKind_t coll = ucclCollAllReduce;
  size_t bytes = 0;        // message size as the bus-bandwidth formulas define it
  int nranks = 1;
  bool nvls = false;       // multicast alias available for the buffers involved
  bool symmetric = false;  // user buffers are symmetric (zero-copy possible)
  bool reducible = true;   // dtype can be reduced (false for fp8 / raw bytes)
  bool netOnly = false;    // no NVLink domain: only the network ring is possible
  bool copyEngine = false; // UCCL_EXEC_MODE=copy_engine
  ucclAlgo_t forcedAlgo = ucclAlgoAuto;
  ucclProto_t forcedProto = ucclProtoAuto;
  int maxBlocks = 0;       // 0 = library limit
};

class Tuner {
 public:
  void clear() { curves_.clear(); tableRanks_ = 0; }
  bool loadFile(const std::string& path, std::string* why);
  bool loadText(const std::string& json, std::string* why);
  // Looks through the *.json tables of `dir` for one measured on this kind of machine: its "gpu"
  // names the device (either string contains the other), "nranks" equals `nranks` and, if the
  // table says so, "nvls" equals `nvls`.  Loads the first match (names in sorted order) and
  // reports its path; false when there is none.
  bool loadMatching(const std::string& dir, const std::string& gpuName, int nranks, bool nvls, std::string* chosen);
  // The three header fields of a table, without loading it.
  static bool tableHeader(const std::string& json, std::string* gpu, int* nranks, int* nvls);
  void addPoint(ucclCollKind_t coll, ucclAlgo_t algo, ucclProto_t proto, size_t bytes, float us, int blocks);
  TuneChoice choose(const TuneQuery& q) const;
  size_t numCurves() const { return curves_.size(); }
  int tableRanks() const { return tableRanks_; }
  // Interpolated time of a curve at `bytes` (log-log), <0 if the curve has no points.
  static float predictUs(const TuneCurve& c, size_t bytes, int* blocks);
  // Is (algo, proto) able to run this query at all?
  static bool feasible(const TuneQuery& q, ucclAlgo_t algo, ucclProto_t proto);

 private:
  TuneChoice prior(const TuneQuery& q) const;
  std::vector<TuneCurve> curves_;
  int tableRanks_ = 0;
};

const char* collName(ucclCollKind_t k);
bool parseColl(const char* s, ucclCollKind_t* out);

}  // namespace uccl
