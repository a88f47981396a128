#include "tuner.h"

#include <ctype.h>
#include <dirent.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>

#include <algorithm>
#include <map>

#include "../kernels/device_comm.h"
#include "config.h"
#include "log.h"

namespace uccl {

const char* collName(ucclCollKind_t k) {
  switch (k) {
    case ucclCollAllReduce: return "allreduce";
    case ucclCollAllGather: return "allgather";
    case ucclCollReduceScatter: return "reducescatter";
    case ucclCollBroadcast: return "broadcast";
    case ucclCollReduce: return "reduce";
    case ucclCollAllToAll: return "alltoall";
    case ucclCollSendRecv: return "sendrecv";
    case ucclCollRma: return "rma";
  }
  return "?";
}

bool parseColl(const char* s, ucclCollKind_t* out) {
  for (int k = 0; k < 8; ++k)
    if (!strcasecmp(s, collName(static_cast<ucclCollKind_t>(k)))) {
      *out = static_cast<ucclCollKind_t>(k);
      return true;
    }
  if (!strcasecmp(s, "reduce_scatter")) { *out = ucclCollReduceScatter; return true; }
  if (!strcasecmp(s, "all_reduce")) { *out = ucclCollAllReduce; return true; }
  if (!strcasecmp(s, "all_gather")) { *out = ucclCollAllGather; return true; }
  return false;
}

// ------------------------------------------------------------------ minimal JSON reader
namespace {

struct JValue {
  enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
  double num = 0;
  bool b = false;
  std::string str;
  std::vector<JValue> arr;
  std::vector<std::pair<std::string, JValue>> obj;
  const JValue* get(const char* key) const {
    for (auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

struct JParser {
  const char* p;
  const char* end;
  std::string err;
  void ws() { while (p < end && isspace(static_cast<unsigned char>(*p))) ++p; }
  bool fail(const char* m) { if (err.empty()) err = m; return false; }
  bool parse(JValue* v) {
    ws();
    if (p >= end) return fail("unexpected end");
    if (*p == '{') {
      v->kind = JValue::OBJ;
      ++p; ws();
      if (p < end && *p == '}') { ++p; return true; }
      while (true) {
        ws();
        JValue k;
        if (p >= end || *p != '"' || !parseString(&k.str)) return fail("object key expected");
        ws();
        if (p >= end || *p != ':') return fail("':' expected");
        ++p;
        JValue val;
        if (!parse(&val)) return false;
        v->obj.emplace_back(k.str, std::move(val));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == '}') { ++p; return true; }
        return fail("',' or '}' expected");
      }
    }
    if (*p == '[') {
      v->kind = JValue::ARR;
      ++p; ws();
      if (p < end && *p == ']') { ++p; return true; }
      while (true) {
        JValue e;
        if (!parse(&e)) return false;
        v->arr.push_back(std::move(e));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == ']') { ++p; return true; }
        return fail("',' or ']' expected");
      }
    }
    if (*p == '"') { v->kind = JValue::STR; return parseString(&v->str); }
    if (!strncmp(p, "true", 4) && end - p >= 4) { v->kind = JValue::BOOL; v->b = true; p += 4; return true; }
    if (!strncmp(p, "false", 5) && end - p >= 5) { v->kind = JValue::BOOL; v->b = false; p += 5; return true; }
    if (!strncmp(p, "null", 4) && end - p >= 4) { v->kind = JValue::NUL; p += 4; return true; }
    char* e = nullptr;
    double d = strtod(p, &e);
    if (e == p) return fail("value expected");
    v->kind = JValue::NUM;
    v->num = d;
    p = e;
    return true;
  }
  bool parseString(std::string* out) {
    ++p;  // opening quote
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          default: out->push_back(*p); break;
        }
        ++p;
      } else {
        out->push_back(*p++);
      }
    }
    if (p >= end) return fail("unterminated string");
    ++p;
    return true;
  }
};

}  // namespace

bool Tuner::loadText(const std::string& json, std::string* why) {
  JParser ps{json.data(), json.data() + json.size(), ""};
  JValue root;
  if (!ps.parse(&root) || root.kind != JValue::OBJ) {
    if (why) *why = ps.err.empty() ? "top-level object expected" : ps.err;
    return false;
  }
  const JValue* entries = root.get("entries");
  if (!entries || entries->kind != JValue::ARR) {
    if (why) *why = "\"entries\" array missing";
    return false;
  }
  std::vector<TuneCurve> fresh;
  std::swap(fresh, curves_);
  curves_.clear();
  size_t added = 0;
  for (const JValue& e : entries->arr) {
    if (e.kind != JValue::OBJ) continue;
    const JValue *c = e.get("coll"), *a = e.get("algo"), *p = e.get("proto"), *b = e.get("bytes"), *u = e.get("us"),
                 *bl = e.get("blocks");
    if (!c || !a || !b || !u || c->kind != JValue::STR || a->kind != JValue::STR || b->kind != JValue::NUM ||
        u->kind != JValue::NUM)
      continue;
    ucclCollKind_t coll;
    ucclAlgo_t algo;
    ucclProto_t proto = ucclProtoSimple;
    if (!parseColl(c->str.c_str(), &coll) || !parseAlgo(a->str.c_str(), &algo)) continue;
    if (p && p->kind == JValue::STR && !parseProto(p->str.c_str(), &proto)) continue;
    if (u->num <= 0 || b->num < 0) continue;
    addPoint(coll, algo, proto, static_cast<size_t>(b->num), static_cast<float>(u->num),
             bl && bl->kind == JValue::NUM ? static_cast<int>(bl->num) : 0);
    ++added;
  }
  if (added == 0) {
    std::swap(fresh, curves_);  // keep what we had
    if (why) *why = "no usable entries";
    return false;
  }
  const JValue* nr = root.get("nranks");
  tableRanks_ = nr && nr->kind == JValue::NUM ? static_cast<int>(nr->num) : 0;
  return true;
}

bool Tuner::loadFile(const std::string& path, std::string* why) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) {
    if (why) *why = "cannot open " + path;
    return false;
  }
  std::string text;
  char buf[4096];
  size_t n;
  while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
  fclose(f);
  return loadText(text, why);
}

namespace {
bool readAll(const std::string& path, std::string* text) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) return false;
  char buf[4096];
  size_t n;
  while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text->append(buf, n);
  fclose(f);
  return true;
}
}  // namespace

bool Tuner::tableHeader(const std::string& json, std::string* gpu, int* nranks, int* nvls) {
  JParser ps{json.data(), json.data() + json.size(), ""};
  JValue root;
  if (!ps.parse(&root) || root.kind != JValue::OBJ) return false;
  const JValue *g = root.get("gpu"), *n = root.get("nranks"), *v = root.get("nvls");
  *gpu = g && g->kind == JValue::STR ? g->str : "";
  *nranks = n && n->kind == JValue::NUM ? static_cast<int>(n->num) : 0;
  *nvls = !v ? -1 : (v->kind == JValue::BOOL ? (v->b ? 1 : 0) : (v->kind == JValue::NUM ? (v->num != 0 ? 1 : 0) : -1));
  return true;
}

bool Tuner::loadMatching(const std::string& dir, const std::string& gpuName, int nranks, bool nvls, std::string* chosen) {
  DIR* d = opendir(dir.c_str());
  if (!d) return false;
  std::vector<std::string> names;
  while (dirent* e = readdir(d)) {
    const std::string n = e->d_name;
    if (n.size() > 5 && n.compare(n.size() - 5, 5, ".json") == 0) names.push_back(n);
  }
  closedir(d);
  std::sort(names.begin(), names.end());
  for (const std::string& n : names) {
    const std::string path = dir + "/" + n;
    std::string text, gpu;
    int ranks = 0, tv = -1;
    if (!readAll(path, &text) || !tableHeader(text, &gpu, &ranks, &tv)) continue;
    if (gpu.empty() || ranks != nranks) continue;
    if (gpuName.find(gpu) == std::string::npos && gpu.find(gpuName) == std::string::npos) continue;
    if (tv >= 0 && (tv != 0) != nvls) continue;
    std::string why;
    if (!loadText(text, &why)) continue;
    if (chosen) *chosen = path;
    return true;
  }
  return false;
}

void Tuner::addPoint(ucclCollKind_t coll, ucclAlgo_t algo, ucclProto_t proto, size_t bytes, float us, int blocks) {
  TuneCurve* cur = nullptr;
  for (auto& c : curves_)
    if (c.coll == coll && c.algo == algo && c.proto == proto) cur = &c;
  if (!cur) {
    curves_.push_back(TuneCurve{coll, algo, proto, {}});
    cur = &curves_.back();
  }
  TunePoint pt{bytes, us, blocks};
  auto it = std::lower_bound(cur->pts.begin(), cur->pts.end(), pt,
                             [](const TunePoint& a, const TunePoint& b) { return a.bytes < b.bytes; });
  if (it != cur->pts.end() && it->bytes == bytes) {
    if (us < it->us) *it = pt;  // keep the best configuration measured for that size
  } else {
    cur->pts.insert(it, pt);
  }
}

float Tuner::predictUs(const TuneCurve& c, size_t bytes, int* blocks) {
  if (c.pts.empty()) return -1.f;
  if (bytes <= c.pts.front().bytes) {
    if (blocks) *blocks = c.pts.front().blocks;
    return c.pts.front().us;
  }
  if (bytes >= c.pts.back().bytes) {
    // extrapolate at the bandwidth of the last point
    if (blocks) *blocks = c.pts.back().blocks;
    const TunePoint& l = c.pts.back();
    return l.bytes ? l.us * static_cast<float>(static_cast<double>(bytes) / static_cast<double>(l.bytes)) : l.us;
  }
  for (size_t i = 1; i < c.pts.size(); ++i) {
    if (bytes <= c.pts[i].bytes) {
      const TunePoint& a = c.pts[i - 1];
      const TunePoint& b = c.pts[i];
      const double la = log(static_cast<double>(std::max<size_t>(a.bytes, 1))), lb = log(static_cast<double>(b.bytes));
      const double t = (log(static_cast<double>(bytes)) - la) / (lb - la);
      if (blocks) *blocks = t < 0.5 ? a.blocks : b.blocks;
      return static_cast<float>(exp(log(a.us) * (1 - t) + log(b.us) * t));
    }
  }
  return c.pts.back().us;
}

bool Tuner::feasible(const TuneQuery& q, ucclAlgo_t algo, ucclProto_t proto) {
  if (q.netOnly) return algo == ucclAlgoNet || algo == ucclAlgoRing;
  if (algo == ucclAlgoNet) return false;
  if (algo == ucclAlgoNvls && !q.nvls) return false;
  if (algo == ucclAlgoNvls && q.coll == ucclCollAllToAll) return false;
  if (algo == ucclAlgoNvls && q.coll == ucclCollSendRecv) return false;
  const bool reduces = q.coll == ucclCollAllReduce || q.coll == ucclCollReduceScatter || q.coll == ucclCollReduce;
  if (reduces && !q.reducible) return false;
  if (proto == ucclProtoLL || proto == ucclProtoLL128) {
    // low-latency protocols: bounded by the per-CTA LL capacity (per message for the all-reduce,
    // per rank chunk for all-gather and reduce-scatter, whose packets exist in the LL form only)
    const bool chunked = q.coll == ucclCollAllGather || q.coll == ucclCollReduceScatter || q.coll == ucclCollAllToAll;
    if (q.coll != ucclCollAllReduce && !(chunked && proto == ucclProtoLL && algo == ucclAlgoOneShot)) return false;
    if (algo != ucclAlgoOneShot && algo != ucclAlgoRing) return false;
    const size_t unit = chunked ? q.bytes / static_cast<size_t>(std::max(q.nranks, 1)) : q.bytes;
    if (unit > static_cast<size_t>(kLLBlocks) * kLLDataPerBlock) return false;
  }
  if (algo == ucclAlgoRing &&
      !(q.coll == ucclCollAllReduce || q.coll == ucclCollAllGather || q.coll == ucclCollReduceScatter))
    return false;
  if (algo == ucclAlgoCopyEngine &&
      !(q.coll == ucclCollAllReduce || q.coll == ucclCollAllGather || q.coll == ucclCollReduceScatter))
    return false;
  return true;
}

static int blocksForBytes(size_t bytes, int nranks) {
  // One CTA per ~256 KiB of per-rank work, between 1 and 64.  Measured on 8 x B200: every CTA runs
  // its own cross-rank barrier, so more CTAs than this made the 1-64 MiB range slower (all-reduce
  // 64 MiB: 175 us with 32 CTAs, 219 us with 64; all-gather 4 MiB: 25 us with 2, 39 us with 16).
  const size_t per = bytes / static_cast<size_t>(std::max(nranks, 1));
  int b = static_cast<int>((per + (256u << 10) - 1) / (256u << 10));
  if (bytes <= (16u << 10)) b = 1;
  else if (bytes <= (256u << 10)) b = std::max(b, 4);
  return std::min(std::max(b, 1), 64);
}

TuneChoice Tuner::prior(const TuneQuery& q) const {
  TuneChoice c;
  c.blocks = blocksForBytes(q.bytes, q.nranks);
  // Without the switch every byte is a peer load or store issued by an SM: one CTA per 64 KiB of
  // per-rank work (2 GPUs, 1 MiB all-reduce: 98 us with 2 CTAs against 22 us for the library).
  if (!(q.nvls && q.nranks > 2) && q.bytes > (64u << 10)) {
    const size_t per = q.bytes / static_cast<size_t>(std::max(q.nranks, 1));
    c.blocks = static_cast<int>(std::min<size_t>(96, std::max<size_t>(c.blocks, (per + (64u << 10) - 1) / (64u << 10))));
  }
  if (q.netOnly) {
    c.algo = ucclAlgoNet;
    c.proto = ucclProtoSimple;
    return c;
  }
  if (q.copyEngine && feasible(q, ucclAlgoCopyEngine, ucclProtoSimple)) {
    c.algo = ucclAlgoCopyEngine;
    return c;
  }
  c.proto = ucclProtoSimple;
  // Between two GPUs the switch has nothing to reduce or replicate and multimem sends this rank's
  // own contribution over the links as well: the fused norm measured 630 us through the switch
  // against 369 us with plain peer accesses for the same 128 MiB.
  const bool nvls = q.nvls && q.nranks > 2;
  switch (q.coll) {
    case ucclCollAllReduce:
      if (q.bytes <= (32u << 10) && feasible(q, ucclAlgoOneShot, ucclProtoLL)) {
        c.algo = ucclAlgoOneShot;
        c.proto = ucclProtoLL;
        c.blocks = static_cast<int>(std::min<size_t>(kLLBlocks, std::max<size_t>(1, (q.bytes + kLLDataPerBlock - 1) / kLLDataPerBlock)));
      } else if (q.bytes <= (256u << 10)) {
        c.algo = ucclAlgoOneShot;
      } else {
        c.algo = nvls ? ucclAlgoNvls : ucclAlgoTwoShot;
      }
      break;
    case ucclCollAllGather:
    case ucclCollReduceScatter:
      // up to 32 KiB per rank the packet form, which needs no barrier at all, wins (2 GPUs: 7 us
      // against 11-13 us for the barrier kernels and 16-21 us for the library, 1 KiB - 64 KiB)
      if (q.bytes / static_cast<size_t>(std::max(q.nranks, 1)) <= (32u << 10) && feasible(q, ucclAlgoOneShot, ucclProtoLL)) {
        c.algo = ucclAlgoOneShot;
        c.proto = ucclProtoLL;
        const size_t chunk = q.bytes / static_cast<size_t>(std::max(q.nranks, 1));
        c.blocks = static_cast<int>(std::min<size_t>(kLLBlocks, std::max<size_t>(1, (chunk + kLLDataPerBlock - 1) / kLLDataPerBlock)));
        break;
      }
      c.algo = (nvls && q.bytes > (64u << 10)) ? ucclAlgoNvls : ucclAlgoTwoShot;
      break;
    case ucclCollBroadcast:
    case ucclCollReduce:
      c.algo = (nvls && q.bytes > (64u << 10)) ? ucclAlgoNvls : ucclAlgoTwoShot;
      if (q.coll == ucclCollReduce && !nvls) c.algo = ucclAlgoOneShot;
      break;
    case ucclCollAllToAll:
      if (q.bytes / static_cast<size_t>(std::max(q.nranks, 1)) <= (32u << 10) && feasible(q, ucclAlgoOneShot, ucclProtoLL)) {
        c.algo = ucclAlgoOneShot;
        c.proto = ucclProtoLL;
        const size_t chunk = q.bytes / static_cast<size_t>(std::max(q.nranks, 1));
        c.blocks = static_cast<int>(std::min<size_t>(kLLBlocks, std::max<size_t>(1, (chunk + kLLDataPerBlock - 1) / kLLDataPerBlock)));
        break;
      }
      // pure copies, nothing to reduce: one CTA per 128 KiB of the message
      c.algo = ucclAlgoTwoShot;
      c.blocks = static_cast<int>(std::min<size_t>(48, std::max<size_t>(c.blocks, q.bytes >> 17)));
      break;
    default:
      c.algo = ucclAlgoTwoShot;
      break;
  }
  return c;
}

TuneChoice Tuner::choose(const TuneQuery& q) const {
  TuneChoice best = prior(q);
  const bool algoForced = q.forcedAlgo != ucclAlgoAuto;
  const bool protoForced = q.forcedProto != ucclProtoAuto;
  float bestUs = -1.f;
  bool found = false;
  for (const TuneCurve& cv : curves_) {
    if (cv.coll != q.coll) continue;
    if (algoForced && cv.algo != q.forcedAlgo) continue;
    if (protoForced && cv.proto != q.forcedProto) continue;
    if (!feasible(q, cv.algo, cv.proto)) continue;
    int blocks = 0;
    const float us = predictUs(cv, q.bytes, &blocks);
    if (us < 0) continue;
    if (!found || us < bestUs) {
      found = true;
      bestUs = us;
      best.algo = cv.algo;
      best.proto = cv.proto;
      if (blocks > 0) best.blocks = blocks;
      best.fromTable = true;
    }
  }
  // a table measured before an algorithm existed does not veto it: the packet form of all-gather /
  // reduce-scatter takes its prior unless the table has a curve for it
  if (found && !algoForced && !protoForced &&
      (q.coll == ucclCollAllGather || q.coll == ucclCollReduceScatter || q.coll == ucclCollAllToAll)) {
    const TuneChoice p = prior(q);
    if (p.proto == ucclProtoLL) {
      bool hasCurve = false;
      for (const TuneCurve& cv : curves_)
        if (cv.coll == q.coll && cv.proto == ucclProtoLL) hasCurve = true;
      if (!hasCurve) {
        best = p;
        found = true;
      }
    }
  }
  if (!found) {
    if (algoForced) {
      ucclProto_t p = protoForced ? q.forcedProto : ucclProtoSimple;
      if (feasible(q, q.forcedAlgo, p)) {
        best.algo = q.forcedAlgo;
        best.proto = p;
        if (p == ucclProtoLL || p == ucclProtoLL128)
          best.blocks = static_cast<int>(std::min<size_t>(kLLBlocks, std::max<size_t>(1, (q.bytes + kLLDataPerBlock - 1) / kLLDataPerBlock)));
      }
    } else if (protoForced && feasible(q, best.algo, q.forcedProto)) {
      best.proto = q.forcedProto;
    }
  }
  int cap = q.maxBlocks > 0 ? std::min(q.maxBlocks, kMaxBlocks) : kMaxBlocks;
  if (best.proto == ucclProtoLL || best.proto == ucclProtoLL128) cap = std::min(cap, kLLBlocks);
  best.blocks = std::min(std::max(best.blocks, 1), cap);
  return best;
}

}  // namespace uccl
