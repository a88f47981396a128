// Native unit tests of the host runtime (no GPU needed).  Each test returns an empty string on
// success or a description of the first failed check.
#include "uccl_selftest.h"

#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <cmath>
#include <deque>
#include <functional>
#include <set>
#include <string>
#include <thread>
#include <vector>

#include "host/host_coll.h"
#include "host/ring_schedule.h"
#include "protocols/protocol.h"
#include "transport/net_plugin.h"
#include "core/bootstrap.h"
#include "core/comm.h"
#include "core/config.h"
#include "core/topo.h"
#include "core/tuner.h"

namespace uccl {
namespace {

std::string fmt(const char* f, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, f);
  vsnprintf(buf, sizeof(buf), f, ap);
  va_end(ap);
  return buf;
}
#define EXPECT(cond)                                                   \
  do {                                                                 \
    if (!(cond)) return fmt("%s:%d: check failed: %s", __FILE__, __LINE__, #cond); \
  } while (0)

// ------------------------------------------------------------------ scripted fake plugin
struct FakeReq {
  int id;
  bool isSend;
  size_t size;
  int testsLeft;  // test() says "not done" this many times first
  bool fail;
};
struct FakeNet {
  std::vector<int> postOrder;    // ids in isend/irecv order
  std::vector<int> doneOrder;    // ids in completion order
  int nextId = 0;
  int delay = 0;                 // testsLeft for new requests
  int failPostAt = -1;           // id whose isend/irecv returns an error
  int failTestAt = -1;           // id whose test() returns an error
  int busyPosts = 0;             // this many posts answer ucclInProgress first
  int shortBy = 0;               // receives report this many bytes fewer
  std::set<FakeReq*> live;
};
FakeNet* g_fake = nullptr;

ucclResult_t fkPost(void* comm, void*, size_t size, void*, void** req, bool isSend) {
  FakeNet* f = static_cast<FakeNet*>(comm);
  if (f->busyPosts > 0) {
    --f->busyPosts;
    return ucclInProgress;
  }
  const int id = f->nextId++;
  if (id == f->failPostAt) return ucclRemoteError;
  FakeReq* r = new FakeReq{id, isSend, size, f->delay, id == f->failTestAt};
  f->live.insert(r);
  f->postOrder.push_back(id);
  *req = r;  // never NULL, even when delay == 0 ("completed inside the call")
  return ucclSuccess;
}
ucclResult_t fkIsend(void* c, void* d, size_t s, void* mh, void** r) { return fkPost(c, d, s, mh, r, true); }
ucclResult_t fkIrecv(void* c, void* d, size_t s, void* mh, void** r) { return fkPost(c, d, s, mh, r, false); }
ucclResult_t fkTest(void* request, int* done, int* size) {
  FakeReq* r = static_cast<FakeReq*>(request);
  if (r->fail) {
    g_fake->live.erase(r);
    delete r;
    return ucclRemoteError;
  }
  if (r->testsLeft > 0) {
    --r->testsLeft;
    *done = 0;
    return ucclSuccess;
  }
  *done = 1;
  *size = static_cast<int>(r->size) - (r->isSend ? 0 : g_fake->shortBy);
  g_fake->doneOrder.push_back(r->id);
  g_fake->live.erase(r);
  delete r;
  return ucclSuccess;
}
ucclResult_t fkNop1(void*) { return ucclSuccess; }

ucclNet_t makeFakeTable() {
  ucclNet_t t;
  memset(&t, 0, sizeof(t));
  t.name = "Fake";
  t.isend = fkIsend;
  t.irecv = fkIrecv;
  t.test = fkTest;
  t.progress = fkNop1;
  return t;
}

struct FakeConn {
  ConnFifo fifo;
  std::vector<char> bounce;
  NetConn conn;
  FakeNet net;
  explicit FakeConn(bool isSend) : bounce(UCCL_STEPS * 1024) {
    memset(&fifo, 0, sizeof(fifo));
    conn.isSend = isSend;
    conn.fifo = &fifo;
    conn.fifoDev = &fifo;
    conn.bounce = bounce.data();
    conn.bounceDev = bounce.data();
    conn.slotBytes = 1024;
    conn.netComm = &net;
    g_fake = &net;
  }
  void post(uint32_t op, size_t bytes) {
    const uint64_t t = fifo.tail;
    FifoEntry& e = fifo.entries[t % UCCL_STEPS];
    e.op = op;
    e.slot = static_cast<uint32_t>(t % UCCL_STEPS);
    e.bytes = bytes;
    e.step = t;
    fifoStoreRelease(&fifo.tail, t + 1);
  }
};

std::string testProxyInOrder() {
  ucclNet_t tab = makeFakeTable();
  FakeConn fc(true);
  fc.net.delay = 3;
  for (int i = 0; i < 5; ++i) fc.post(FIFO_SEND, 100 + i);
  uint64_t posts = 0, comps = 0;
  for (int pass = 0; pass < 40 && fc.fifo.head < 5; ++pass)
    EXPECT(proxyProgressConn(&tab, &fc.conn, &posts, &comps) == ucclSuccess);
  EXPECT(fc.fifo.head == 5);
  EXPECT(posts == 5 && comps == 5);
  EXPECT(fc.net.postOrder == std::vector<int>({0, 1, 2, 3, 4}));
  EXPECT(fc.net.doneOrder == std::vector<int>({0, 1, 2, 3, 4}));
  EXPECT(fc.fifo.entries[2].result == 102);
  EXPECT(fc.net.live.empty());
  return "";
}

// An operation that completes inside isend() must be posted exactly once (the reference
// re-posts it because it keys "posted" on a non-NULL request, src/proxy.cc:37-76 with
// src/plugin/net_ucx.cc:378-381).
std::string testProxyImmediateCompletion() {
  ucclNet_t tab = makeFakeTable();
  FakeConn fc(true);
  fc.net.delay = 0;
  for (int i = 0; i < UCCL_STEPS; ++i) fc.post(FIFO_SEND, 64);
  uint64_t posts = 0, comps = 0;
  for (int pass = 0; pass < 5; ++pass) EXPECT(proxyProgressConn(&tab, &fc.conn, &posts, &comps) == ucclSuccess);
  EXPECT(fc.net.postOrder.size() == static_cast<size_t>(UCCL_STEPS));
  EXPECT(posts == UCCL_STEPS && comps == UCCL_STEPS);
  EXPECT(fc.fifo.head == UCCL_STEPS);
  // more work after the ring wrapped
  for (int i = 0; i < 3; ++i) fc.post(FIFO_SEND, 32);
  for (int pass = 0; pass < 5; ++pass) EXPECT(proxyProgressConn(&tab, &fc.conn, &posts, &comps) == ucclSuccess);
  EXPECT(fc.net.postOrder.size() == static_cast<size_t>(UCCL_STEPS + 3));
  EXPECT(fc.fifo.head == UCCL_STEPS + 3);
  return "";
}

std::string testProxyBusyAndSignal() {
  ucclNet_t tab = makeFakeTable();
  FakeConn fc(true);
  fc.net.busyPosts = 2;  // plugin out of resources twice
  fc.post(FIFO_SIGNAL, 0);
  fc.post(FIFO_PUT, 10);
  uint64_t posts = 0, comps = 0;
  EXPECT(proxyProgressConn(&tab, &fc.conn, &posts, &comps) == ucclSuccess);
  EXPECT(posts == 0);
  EXPECT(proxyProgressConn(&tab, &fc.conn, &posts, &comps) == ucclSuccess);
  EXPECT(posts == 0);
  for (int pass = 0; pass < 4; ++pass) EXPECT(proxyProgressConn(&tab, &fc.conn, &posts, &comps) == ucclSuccess);
  EXPECT(posts == 2 && comps == 2 && fc.fifo.head == 2);
  EXPECT(fc.fifo.entries[0].result == 0);
  return "";
}

std::string testProxyErrors() {
  ucclNet_t tab = makeFakeTable();
  {
    FakeConn fc(false);
    fc.net.failPostAt = 1;
    for (int i = 0; i < 3; ++i) fc.post(FIFO_RECV, 128);
    uint64_t posts = 0, comps = 0;
    ucclResult_t r = proxyProgressConn(&tab, &fc.conn, &posts, &comps);
    EXPECT(r == ucclRemoteError);
    EXPECT(fc.fifo.error == static_cast<uint64_t>(ucclRemoteError));
    EXPECT(posts == 1);
    // latched: later passes neither post nor complete anything
    EXPECT(proxyProgressConn(&tab, &fc.conn, &posts, &comps) == ucclSuccess);
    EXPECT(posts == 1);
    for (FakeReq* r2 : fc.net.live) delete r2;
  }
  {
    FakeConn fc(false);
    fc.net.failTestAt = 0;
    fc.post(FIFO_RECV, 128);
    uint64_t posts = 0, comps = 0;
    EXPECT(proxyProgressConn(&tab, &fc.conn, &posts, &comps) == ucclRemoteError);
    EXPECT(fc.fifo.head == 0 && fc.fifo.error != 0);
  }
  {
    // short read is reported through `result`, the consumer decides
    FakeConn fc(false);
    fc.net.shortBy = 8;
    fc.post(FIFO_RECV, 128);
    uint64_t posts = 0, comps = 0;
    for (int pass = 0; pass < 3; ++pass) EXPECT(proxyProgressConn(&tab, &fc.conn, &posts, &comps) == ucclSuccess);
    EXPECT(fc.fifo.head == 1 && fc.fifo.entries[0].result == 120);
  }
  return "";
}

// ------------------------------------------------------------------ LL128 codec
std::string testLL128() {
  for (size_t bytes : {size_t(0), size_t(1), size_t(111), size_t(112), size_t(113), size_t(1000), size_t(4096)}) {
    std::vector<unsigned char> src(bytes), dst(bytes, 0xEE);
    for (size_t i = 0; i < bytes; ++i) src[i] = static_cast<unsigned char>(i * 7 + 3);
    const size_t lines = ll128LinesFor(bytes);
    std::vector<uint64_t> buf((lines + 1) * ProtoLL128::LineElems, 0);
    EXPECT(ll128ProtocolSend(buf.data(), buf.size() * 8, src.data(), bytes, 5) == ucclSuccess);
    for (size_t l = 0; l < lines; ++l) {
      EXPECT(buf[l * 16 + 7] == 5 && buf[l * 16 + 15] == 5);
    }
    EXPECT(ll128ProtocolRecv(buf.data(), buf.size() * 8, dst.data(), bytes, 5, 10) == ucclSuccess);
    EXPECT(src == dst);
    // a stale sequence number must not validate
    if (bytes) EXPECT(ll128ProtocolRecv(buf.data(), buf.size() * 8, dst.data(), bytes, 6, 100) == ucclRemoteError);
  }
  // a half-written line (one flag only) is not valid
  uint64_t line[16] = {0};
  unsigned char payload[112] = {1, 2, 3};
  ll128PackLine(line, payload, 112, 9);
  line[15] = 8;
  unsigned char out[112];
  EXPECT(!ll128UnpackLine(line, out, 112, 9, 50));
  EXPECT(ll128ProtocolSend(line, 64, payload, 112, 1) == ucclInvalidArgument);  // buffer too small
  EXPECT(ll128ProtocolSend(line, 128, payload, 112, 0) == ucclInvalidArgument); // seq 0 is reserved
  return "";
}

// ------------------------------------------------------------------ ring schedule vs brute force
std::string testRingSchedule() {
  for (int n = 1; n <= 16; ++n) {
    for (size_t count : {size_t(0), size_t(1), size_t(n - 1), size_t(n), size_t(n + 1), size_t(5 * n + 3), size_t(1000)}) {
      // chunks tile [0, count) without gaps
      size_t expectOff = 0;
      for (int c = 0; c < n; ++c) {
        size_t off, len;
        ringChunk(count, n, c, &off, &len);
        EXPECT(off == expectOff);
        expectOff += len;
      }
      EXPECT(expectOff == count);
      // have[r][c] = set of ranks whose contribution to chunk c rank r holds
      std::vector<std::vector<uint32_t>> have(n, std::vector<uint32_t>(n));
      for (int r = 0; r < n; ++r)
        for (int c = 0; c < n; ++c) have[r][c] = 1u << r;
      for (int s = 0; s < n - 1; ++s) {
        std::vector<std::vector<uint32_t>> next = have;
        for (int r = 0; r < n; ++r) {
          const int to = (r + 1) % n;
          const int sc = ringRsSendChunk(r, s, n);
          EXPECT(ringRsRecvChunk(to, s, n) == sc);  // what I send is what my successor expects
          next[to][sc] = have[to][sc] | have[r][sc];
        }
        have = next;
      }
      const uint32_t all = n == 32 ? 0xffffffffu : ((1u << n) - 1);
      for (int r = 0; r < n; ++r) EXPECT(have[r][(r + 1) % n] == all);
      for (int s = 0; s < n - 1; ++s) {
        std::vector<std::vector<uint32_t>> next = have;
        for (int r = 0; r < n; ++r) {
          const int to = (r + 1) % n;
          const int sc = ringAgSendChunk(r, s, n);
          EXPECT(ringAgRecvChunk(to, s, n) == sc);
          EXPECT(have[r][sc] == all);  // only complete chunks are forwarded
          next[to][sc] = have[r][sc];
        }
        have = next;
      }
      for (int r = 0; r < n; ++r)
        for (int c = 0; c < n; ++c) EXPECT(have[r][c] == all);
    }
  }
  return "";
}

// ------------------------------------------------------------------ tuner
std::string testTuner() {
  Tuner t;
  TuneQuery q;
  q.coll = ucclCollAllReduce;
  q.nranks = 8;
  q.nvls = true;
  q.bytes = 1024;
  TuneChoice c = t.choose(q);
  EXPECT(c.algo == ucclAlgoOneShot && c.proto == ucclProtoLL && !c.fromTable);
  q.bytes = 64u << 20;
  c = t.choose(q);
  EXPECT(c.algo == ucclAlgoNvls);
  q.nranks = 2;  // the switch brings nothing between two GPUs
  c = t.choose(q);
  EXPECT(c.algo == ucclAlgoTwoShot);
  q.nranks = 8;
  q.nvls = false;
  c = t.choose(q);
  EXPECT(c.algo == ucclAlgoTwoShot);
  q.netOnly = true;
  c = t.choose(q);
  EXPECT(c.algo == ucclAlgoNet);
  q.netOnly = false;
  q.forcedAlgo = ucclAlgoRing;
  c = t.choose(q);
  EXPECT(c.algo == ucclAlgoRing && c.proto == ucclProtoSimple);
  q.forcedAlgo = ucclAlgoNvls;  // not feasible without multicast: falls back to the prior
  c = t.choose(q);
  EXPECT(c.algo == ucclAlgoTwoShot);
  q.forcedAlgo = ucclAlgoAuto;

  const char* json =
      "{\"version\":1,\"nranks\":8,\"entries\":["
      "{\"coll\":\"allreduce\",\"algo\":\"one_shot\",\"proto\":\"simple\",\"bytes\":1024,\"us\":5.0,\"blocks\":2},"
      "{\"coll\":\"allreduce\",\"algo\":\"one_shot\",\"proto\":\"simple\",\"bytes\":1048576,\"us\":60.0,\"blocks\":16},"
      "{\"coll\":\"allreduce\",\"algo\":\"two_shot\",\"proto\":\"simple\",\"bytes\":1024,\"us\":9.0,\"blocks\":2},"
      "{\"coll\":\"allreduce\",\"algo\":\"two_shot\",\"proto\":\"simple\",\"bytes\":1048576,\"us\":20.0,\"blocks\":32},"
      "{\"coll\":\"allreduce\",\"algo\":\"nvls\",\"proto\":\"simple\",\"bytes\":1048576,\"us\":10.0,\"blocks\":24},"
      "{\"coll\":\"bogus\",\"algo\":\"nvls\",\"bytes\":1,\"us\":1}"
      "]}";
  std::string why;
  EXPECT(t.loadText(json, &why));
  EXPECT(t.numCurves() == 3 && t.tableRanks() == 8);
  q.bytes = 2048;
  c = t.choose(q);
  EXPECT(c.fromTable && c.algo == ucclAlgoOneShot && c.blocks == 2);
  q.bytes = 1u << 20;
  c = t.choose(q);
  EXPECT(c.algo == ucclAlgoTwoShot && c.blocks == 32);  // NVLS curve exists but is not feasible
  q.nvls = true;
  c = t.choose(q);
  EXPECT(c.algo == ucclAlgoNvls && c.blocks == 24);
  q.maxBlocks = 4;
  c = t.choose(q);
  EXPECT(c.blocks == 4);
  q.maxBlocks = 0;
  // interpolation is monotone between the two one-shot points
  TuneCurve cv{ucclCollAllReduce, ucclAlgoOneShot, ucclProtoSimple, {{1024, 5.f, 2}, {1048576, 60.f, 16}}};
  int blocks = 0;
  const float mid = Tuner::predictUs(cv, 32768, &blocks);
  EXPECT(mid > 5.f && mid < 60.f);
  EXPECT(std::fabs(Tuner::predictUs(cv, 2u << 20, &blocks) - 120.f) < 1e-3f);  // bandwidth extrapolation
  EXPECT(!t.loadText("{\"entries\":[]}", &why));
  EXPECT(!t.loadText("not json", &why));
  EXPECT(t.numCurves() == 3);  // a rejected table leaves the old one in place
  // shipped tables are matched by GPU name, rank count and NVLS flag
  {
    char dir[] = "/tmp/uccl_tune_XXXXXX";
    EXPECT(mkdtemp(dir) != nullptr);
    auto put = [&](const char* name, const char* gpu, int ranks, const char* nvls, double us) {
      const std::string path = std::string(dir) + "/" + name;
      FILE* f = fopen(path.c_str(), "w");
      if (!f) return;
      fprintf(f, "{\"version\":1,\"gpu\":\"%s\",\"nranks\":%d%s,\"entries\":[{\"coll\":\"allreduce\",\"algo\":\"two_shot\","
                 "\"proto\":\"simple\",\"bytes\":4096,\"us\":%f,\"blocks\":3}]}", gpu, ranks, nvls, us);
      fclose(f);
    };
    put("a_other_gpu.json", "NVIDIA H100", 8, "", 1.0);
    put("b_b200_x4.json", "NVIDIA B200", 4, "", 2.0);
    put("c_b200_x8_nonvls.json", "NVIDIA B200", 8, ",\"nvls\":false", 3.0);
    put("d_b200_x8.json", "NVIDIA B200", 8, ",\"nvls\":true", 4.0);
    put("e_not_a_table.json", "NVIDIA B200", 8, "", -1.0);
    Tuner m;
    std::string chosen;
    EXPECT(m.loadMatching(dir, "NVIDIA B200", 8, true, &chosen));
    EXPECT(chosen.find("d_b200_x8.json") != std::string::npos && m.tableRanks() == 8);
    EXPECT(m.loadMatching(dir, "NVIDIA B200", 8, false, &chosen) && chosen.find("c_b200_x8_nonvls") != std::string::npos);
    EXPECT(m.loadMatching(dir, "NVIDIA B200", 4, true, &chosen) && chosen.find("b_b200_x4") != std::string::npos);
    EXPECT(!m.loadMatching(dir, "NVIDIA B200", 2, true, &chosen));
    EXPECT(!m.loadMatching(dir, "NVIDIA A100", 8, true, &chosen));
    EXPECT(!m.loadMatching(std::string(dir) + "/missing", "NVIDIA B200", 8, true, &chosen));
    std::string gpu;
    int ranks = 0, nv = 0;
    EXPECT(Tuner::tableHeader("{\"gpu\":\"X\",\"nranks\":2}", &gpu, &ranks, &nv) && gpu == "X" && ranks == 2 && nv == -1);
    for (const char* n : {"a_other_gpu.json", "b_b200_x4.json", "c_b200_x8_nonvls.json", "d_b200_x8.json", "e_not_a_table.json"})
      unlink((std::string(dir) + "/" + n).c_str());
    rmdir(dir);
  }
  // reductions on a type that cannot be summed are never offered
  q.reducible = false;
  EXPECT(!Tuner::feasible(q, ucclAlgoTwoShot, ucclProtoSimple));
  q.coll = ucclCollAllGather;
  EXPECT(Tuner::feasible(q, ucclAlgoTwoShot, ucclProtoSimple));
  EXPECT(!Tuner::feasible(q, ucclAlgoOneShot, ucclProtoLL));
  // the packet form of the chunked collectives: feasible up to 64 KiB per rank, the prior up to 32 KiB,
  // and a table that was measured without it does not veto it
  {
    TuneQuery g;
    g.coll = ucclCollAllGather;
    g.nranks = 8;
    g.nvls = true;
    g.bytes = 8u * (64u << 10);
    EXPECT(Tuner::feasible(g, ucclAlgoOneShot, ucclProtoLL));
    g.bytes += 8;
    EXPECT(!Tuner::feasible(g, ucclAlgoOneShot, ucclProtoLL));
    Tuner u;
    g.bytes = 8u * 4096u;
    TuneChoice k = u.choose(g);
    EXPECT(k.algo == ucclAlgoOneShot && k.proto == ucclProtoLL && k.blocks == 1);
    g.bytes = 8u * (48u << 10);
    k = u.choose(g);
    EXPECT(k.proto == ucclProtoSimple);
    std::string w;
    EXPECT(u.loadText("{\"version\":1,\"nranks\":8,\"entries\":["
                      "{\"coll\":\"allgather\",\"algo\":\"two_shot\",\"proto\":\"simple\",\"bytes\":1024,\"us\":12.0,\"blocks\":1},"
                      "{\"coll\":\"allgather\",\"algo\":\"two_shot\",\"proto\":\"simple\",\"bytes\":1048576,\"us\":20.0,\"blocks\":8}]}", &w));
    g.bytes = 8u * 4096u;
    k = u.choose(g);
    EXPECT(k.algo == ucclAlgoOneShot && k.proto == ucclProtoLL);  // no curve for it in the table: the prior stands
    EXPECT(u.loadText("{\"version\":1,\"nranks\":8,\"entries\":["
                      "{\"coll\":\"allgather\",\"algo\":\"two_shot\",\"proto\":\"simple\",\"bytes\":1024,\"us\":12.0,\"blocks\":1},"
                      "{\"coll\":\"allgather\",\"algo\":\"two_shot\",\"proto\":\"simple\",\"bytes\":1048576,\"us\":20.0,\"blocks\":8},"
                      "{\"coll\":\"allgather\",\"algo\":\"one_shot\",\"proto\":\"ll\",\"bytes\":1024,\"us\":30.0,\"blocks\":1},"
                      "{\"coll\":\"allgather\",\"algo\":\"one_shot\",\"proto\":\"ll\",\"bytes\":65536,\"us\":40.0,\"blocks\":2}]}", &w));
    k = u.choose(g);
    EXPECT(k.fromTable && k.algo == ucclAlgoTwoShot);  // measured slower here: the table decides
    g.coll = ucclCollAllToAll;
    g.bytes = 8u * 1024u;
    Tuner v;
    k = v.choose(g);
    EXPECT(k.algo == ucclAlgoOneShot && k.proto == ucclProtoLL);
  }
  return "";
}

// ------------------------------------------------------------------ plugin loader
std::string testPluginLoader() {
  std::string why;
  EXPECT(loadNetPlugin("", &why) == nullptr);
  EXPECT(loadNetPlugin("../evil.so", &why) == nullptr && why.find("..") != std::string::npos);
  EXPECT(loadNetPlugin("/tmp/plugin.txt", &why) == nullptr && why.find(".so") != std::string::npos);
  EXPECT(loadNetPlugin("/nonexistent/dir/libnothing.so", &why) == nullptr && why.find("dlopen") != std::string::npos);
  // a real shared object without the plugin symbol: this library itself (when the tests are linked
  // into an executable there is no such file and the case is skipped)
  Dl_info info;
  if (dladdr(reinterpret_cast<void*>(&ucclSelfTestCount), &info) && info.dli_fname &&
      strlen(info.dli_fname) > 3 && !strcmp(info.dli_fname + strlen(info.dli_fname) - 3, ".so")) {
    EXPECT(loadNetPlugin(info.dli_fname, &why) == nullptr);
    EXPECT(why.find("ucclNetPlugin_v1") != std::string::npos);
  }
  ucclNet_t* builtin = autoLoadNetPlugin("/nonexistent/dir/libnothing.so");
  EXPECT(builtin == builtinSocketPlugin());
  EXPECT(netPluginComplete(builtin, &why));
  ucclNet_t hole = *builtin;
  hole.setTag = nullptr;
  EXPECT(!netPluginComplete(&hole, &why) && why.find("setTag") != std::string::npos);
  const char* ext = getenv("UCCL_SELFTEST_PLUGIN");
  if (ext && *ext) {
    ucclNet_t* p = loadNetPlugin(ext, &why);
    EXPECT(p != nullptr);
    EXPECT(std::string(p->name) == "UnixSample");
  }
  return "";
}

// ------------------------------------------------------------------ socket plugin loopback
std::string testSocketLoopback() {
  ucclNet_t* net = builtinSocketPlugin();
  void* ctx = nullptr;
  setenv("UCCL_SOCKET_IFNAME", "lo", 0);
  EXPECT(net->init(&ctx) == ucclSuccess);
  int nd = 0;
  EXPECT(net->devices(&nd) == ucclSuccess && nd == 1);
  ucclNetProperties_t props;
  EXPECT(net->getProperties(0, &props) == ucclSuccess && (props.ptrSupport & UCCL_PTR_HOST));
  char handle[UCCL_NET_HANDLE_BYTES];
  void *lc = nullptr, *sc = nullptr, *rc = nullptr;
  EXPECT(net->listen(ctx, handle, &lc) == ucclSuccess);
  EXPECT(net->connect(ctx, handle, &sc) == ucclSuccess);
  for (int i = 0; i < 1000 && !rc; ++i) {
    ucclResult_t r = net->accept(lc, &rc);
    EXPECT(r == ucclSuccess || r == ucclInProgress);
  }
  EXPECT(rc != nullptr);
  net->setTag(sc, 42);
  net->setTag(rc, 42);
  std::vector<char> out(300000), in(300000, 0);
  for (size_t i = 0; i < out.size(); ++i) out[i] = static_cast<char>(i * 13);
  void *mhS = nullptr, *mhR = nullptr;
  EXPECT(net->regMr(sc, out.data(), out.size(), UCCL_PTR_HOST, &mhS) == ucclSuccess);
  EXPECT(net->regMr(rc, in.data(), in.size(), UCCL_PTR_HOST, &mhR) == ucclSuccess);
  EXPECT(net->regMr(rc, in.data(), in.size(), UCCL_PTR_DEVICE, &mhR) == ucclInvalidArgument);
  void *rs = nullptr, *rr = nullptr;
  EXPECT(net->irecv(rc, in.data(), in.size(), mhR, &rr) == ucclSuccess && rr);
  EXPECT(net->isend(sc, out.data(), out.size(), mhS, &rs) == ucclSuccess && rs);
  int ds = 0, dr = 0, sz = 0;
  for (int i = 0; i < 100000 && !(ds && dr); ++i) {
    if (!ds) EXPECT(net->test(rs, &ds, &sz) == ucclSuccess);
    if (!dr) EXPECT(net->test(rr, &dr, &sz) == ucclSuccess);
    net->progress(ctx);
  }
  EXPECT(ds && dr && sz == static_cast<int>(out.size()));
  EXPECT(in == out);
  // zero-byte message (signal)
  EXPECT(net->irecv(rc, in.data(), 16, mhR, &rr) == ucclSuccess);
  EXPECT(net->isend(sc, out.data(), 0, mhS, &rs) == ucclSuccess);
  ds = dr = 0;
  for (int i = 0; i < 100000 && !(ds && dr); ++i) {
    if (!ds) EXPECT(net->test(rs, &ds, &sz) == ucclSuccess);
    if (!dr) EXPECT(net->test(rr, &dr, &sz) == ucclSuccess);
  }
  EXPECT(ds && dr && sz == 0);
  // the receiver notices a vanished sender
  EXPECT(net->irecv(rc, in.data(), 16, mhR, &rr) == ucclSuccess);
  EXPECT(net->closeSend(sc) == ucclSuccess);
  ucclResult_t last = ucclSuccess;
  dr = 0;
  for (int i = 0; i < 100000 && !dr && last == ucclSuccess; ++i) last = net->test(rr, &dr, &sz);
  EXPECT(last == ucclRemoteError);
  EXPECT(net->closeRecv(rc) == ucclSuccess);
  EXPECT(net->closeListen(lc) == ucclSuccess);
  EXPECT(net->finalize(ctx) == ucclSuccess);
  return "";
}

// ------------------------------------------------------------------ topology
std::string testTopology() {
  EXPECT(parseBusId("0000:1b:00.0") == ((0x1b << 12) | 0));
  EXPECT(parseBusId("0001:A3:02.1") == ((int64_t(1) << 20) | (0xa3 << 12) | (2 << 4) | 1));
  EXPECT(parseBusId("garbage") == -1);
  // eight GPUs, two sockets, interleaved device numbering
  TopoSystem sys;
  const int sockets[8] = {0, 1, 0, 1, 0, 1, 0, 1};
  for (int i = 0; i < 8; ++i) {
    TopoGpu g;
    g.dev = i;
    g.rank = i;
    g.busIdNum = (0x10 + 8 * (7 - i)) << 12;
    g.socket = sockets[i];
    g.numaNode = sockets[i];
    sys.gpus.push_back(g);
  }
  std::vector<P2pFacts> pcie(64);
  for (auto& f : pcie) f.access = 1;
  sys.nvswitch = false;
  topoBuildLinks(&sys, pcie);
  EXPECT(sys.allP2p);
  EXPECT(sys.link(0, 1).type == LINK_SYS);
  EXPECT(sys.link(0, 2).type == LINK_PCIE_HOST || sys.link(0, 2).type == LINK_PCIE_SWITCH);
  std::vector<int> order = topoRingOrder(sys);
  EXPECT(order.size() == 8);
  EXPECT(topoSocketCrossings(sys, order) == 2);
  for (int i = 0; i < 3; ++i) {
    EXPECT(sys.gpus[order[i]].socket == 0);
    EXPECT(sys.gpus[order[i]].busIdNum < sys.gpus[order[i + 1]].busIdNum);
  }
  TopoTuning tt = topoTune(sys, 1024);
  EXPECT(tt.algo == ucclAlgoRing && tt.proto == ucclProtoLL128 && tt.nChannels == 8);
  tt = topoTune(sys, 100u << 10);
  EXPECT(tt.proto == ucclProtoSimple);  // crosses sockets
  tt = topoTune(sys, 8u << 20);
  EXPECT(tt.proto == ucclProtoSimple && tt.chunkBytes == (512u << 10));
  EXPECT(tt.bwGBs == 32.f && tt.latUs == 1.0f);  // slowest link, slowest latency
  // the same machine behind an NVSwitch
  std::vector<P2pFacts> nvl(64);
  for (auto& f : nvl) { f.access = 1; f.nativeAtomics = 1; }
  sys.nvswitch = true;
  topoBuildLinks(&sys, nvl);
  EXPECT(sys.link(3, 6).type == LINK_NVSWITCH && sys.link(3, 6).bwGBs == 900.f);
  EXPECT(sys.link(2, 2).type == LINK_SELF);
  tt = topoTune(sys, 1024);
  EXPECT(tt.algo == ucclAlgoOneShot && tt.proto == ucclProtoLL);
  tt = topoTune(sys, 64u << 20);
  EXPECT(tt.algo == ucclAlgoNvls);
  // a pair without peer access disables the NVLink domain
  nvl[1 * 8 + 5].access = 0;
  topoBuildLinks(&sys, nvl);
  EXPECT(!sys.allP2p);
  // small systems
  TopoSystem two;
  two.gpus.resize(2);
  two.gpus[1].dev = 1;
  two.gpus[1].busIdNum = 0x2000;
  std::vector<P2pFacts> f2(4);
  topoBuildLinks(&two, f2);
  EXPECT(topoTune(two, 1u << 20).nChannels == 2);
  return "";
}

// ------------------------------------------------------------------ conversions + reductions
std::string testConversions() {
  EXPECT(bf16ToFloat(0x3f80) == 1.0f);
  EXPECT(floatToBf16(1.0f) == 0x3f80);
  EXPECT(floatToBf16(-2.5f) == 0xc020);
  EXPECT(halfToFloat(0x3c00) == 1.0f);
  EXPECT(floatToHalf(1.0f) == 0x3c00);
  EXPECT(floatToHalf(65504.0f) == 0x7bff);
  EXPECT(floatToHalf(1e6f) == 0x7c00);
  EXPECT(halfToFloat(0x0001) > 0.f && halfToFloat(0x0001) < 1e-7f);
  for (uint32_t h = 0; h < 0x7c00; h += 37) EXPECT(floatToHalf(halfToFloat(static_cast<uint16_t>(h))) == h);
  for (uint32_t b = 0; b < 0x7f80; b += 41) EXPECT(floatToBf16(bf16ToFloat(static_cast<uint16_t>(b))) == b);
  // round to nearest even
  float x;
  uint32_t u = 0x3f808000u;  // exactly half-way between two bf16 values, even mantissa below
  memcpy(&x, &u, 4);
  EXPECT(floatToBf16(x) == 0x3f80);
  u = 0x3f818000u;
  memcpy(&x, &u, 4);
  EXPECT(floatToBf16(x) == 0x3f82);
  float a[4] = {1, 2, 3, 4}, b[4] = {0.5f, 0.25f, -3, 10};
  hostReduceInto(a, b, 4, ucclFloat32);
  EXPECT(a[0] == 1.5f && a[1] == 2.25f && a[2] == 0.f && a[3] == 14.f);
  uint16_t p[2] = {floatToBf16(1.0f), floatToBf16(100.f)}, q[2] = {floatToBf16(2.0f), floatToBf16(0.25f)};
  hostReduceInto(p, q, 2, ucclBfloat16);
  EXPECT(bf16ToFloat(p[0]) == 3.0f && bf16ToFloat(p[1]) == 100.0f);  // 100.25 rounds to 100 in bf16
  EXPECT(dataTypeSize(ucclFloat16) == 2 && dataTypeSize(ucclFloat32) == 4 && dataTypeSize(ucclFloat8e4m3) == 1);
  return "";
}

// ------------------------------------------------------------------ configuration parsing
std::string testConfig() {
  ucclAlgo_t a;
  ucclProto_t p;
  EXPECT(parseAlgo("ring", &a) && a == ucclAlgoRing);
  EXPECT(parseAlgo("ONE_SHOT", &a) && a == ucclAlgoOneShot);
  EXPECT(parseAlgo("symmetric", &a) && a == ucclAlgoTwoShot);
  EXPECT(parseAlgo("ce", &a) && a == ucclAlgoCopyEngine);
  EXPECT(parseAlgo("copy_engine", &a) && a == ucclAlgoCopyEngine);
  EXPECT(parseAlgo("nvls", &a) && a == ucclAlgoNvls);
  EXPECT(!parseAlgo("quantum", &a) && !parseAlgo("", &a));
  EXPECT(parseProto("ll128", &p) && p == ucclProtoLL128);
  EXPECT(parseProto("Simple", &p) && p == ucclProtoSimple);
  EXPECT(!parseProto("fast", &p));
  EXPECT(parseSize("64M", 1) == (64ull << 20));
  EXPECT(parseSize("2g", 1) == (2ull << 30));
  EXPECT(parseSize("512k", 1) == (512ull << 10));
  EXPECT(parseSize("100", 1) == 100);
  EXPECT(parseSize("", 7) == 7 && parseSize("abc", 7) == 7);
  setenv("UCCL_ALGO", "two_shot", 1);
  setenv("UCCL_EXEC_MODE", "ce", 1);
  setenv("UCCL_EU_COUNT", "12", 1);
  setenv("UCCL_FORCE_NET", "1", 1);
  setenv("UCCL_WAIT_TIMEOUT_MS", "1500", 1);
  Config c = loadConfig();
  unsetenv("UCCL_ALGO");
  unsetenv("UCCL_EXEC_MODE");
  unsetenv("UCCL_EU_COUNT");
  unsetenv("UCCL_FORCE_NET");
  unsetenv("UCCL_WAIT_TIMEOUT_MS");
  EXPECT(c.algo == ucclAlgoTwoShot && c.execMode == EXEC_COPY_ENGINE && c.maxCtas == 12 && c.forceNet);
  EXPECT(c.waitTimeoutMs == 1500);
  Config d = loadConfig();
  EXPECT(d.algo == ucclAlgoAuto && d.execMode == EXEC_SM_ONLY && !d.forceNet && d.waitTimeoutMs == 10000);
  // a wait budget of zero, a negative one or an absurd one is clamped: device waits stay bounded
  setenv("UCCL_WAIT_TIMEOUT_MS", "0", 1);
  EXPECT(loadConfig().waitTimeoutMs == 1);
  setenv("UCCL_WAIT_TIMEOUT_MS", "-5", 1);
  EXPECT(loadConfig().waitTimeoutMs == 1);
  setenv("UCCL_WAIT_TIMEOUT_MS", "99999999999", 1);
  EXPECT(loadConfig().waitTimeoutMs == 600000);
  unsetenv("UCCL_WAIT_TIMEOUT_MS");
  return "";
}

// ------------------------------------------------------------------ unique id + API misuse
std::string testApiRules() {
  ucclUniqueId id;
  EXPECT(bootstrapIdFromAddress("127.0.0.1", 23456, 99, &id) == ucclSuccess);
  BootstrapIdPayload p;
  memcpy(&p, id.internal, sizeof(p));
  EXPECT(p.magic == kBootstrapMagic && ntohs(p.addr.sin_port) == 23456);
  ucclUniqueId id2;
  EXPECT(bootstrapIdFromAddress("127.0.0.1", 23456, 99, &id2) == ucclSuccess);
  EXPECT(memcmp(id.internal, id2.internal, UCCL_UNIQUE_ID_BYTES) == 0);  // deterministic: all ranks derive it
  EXPECT(bootstrapIdFromAddress("127.0.0.1", 23456, 100, &id2) == ucclSuccess);
  EXPECT(memcmp(id.internal, id2.internal, UCCL_UNIQUE_ID_BYTES) != 0);
  EXPECT(bootstrapIdFromAddress("not-an-ip", 1, 0, &id2) == ucclInvalidArgument);
  EXPECT(bootstrapIdFromAddress("127.0.0.1", 0, 0, &id2) == ucclInvalidArgument);

  // group depth rules
  EXPECT(ucclGroupEnd() == ucclInvalidUsage);
  EXPECT(ucclGroupStart() == ucclSuccess);
  EXPECT(ucclGroupStart() == ucclSuccess);
  EXPECT(ucclGroupEnd() == ucclSuccess);
  EXPECT(ucclGroupEnd() == ucclSuccess);
  EXPECT(ucclGroupEnd() == ucclInvalidUsage);

  // argument validation without a communicator
  ucclComm_t none = nullptr;
  float x = 0;
  EXPECT(ucclAllReduce(&x, &x, 1, ucclFloat32, ucclSum, none, nullptr) == ucclInvalidArgument);
  EXPECT(ucclCommInitRank(nullptr, 1, id, 0) == ucclInvalidArgument);
  ucclComm_t c = nullptr;
  EXPECT(ucclCommInitRank(&c, 0, id, 0) == ucclInvalidArgument);
  EXPECT(ucclCommInitRank(&c, 2, id, 2) == ucclInvalidArgument);
  EXPECT(ucclCommInitRank(&c, UCCL_MAX_RANKS + 1, id, 0) == ucclInvalidArgument);
  EXPECT(ucclCommDestroy(nullptr) == ucclSuccess);
  int v = 0;
  EXPECT(ucclGetVersion(&v) == ucclSuccess && v == 100);
  EXPECT(ucclGetVersion(nullptr) == ucclInvalidArgument);
  for (int r = 0; r < ucclNumResults; ++r) EXPECT(strlen(ucclGetErrorString(static_cast<ucclResult_t>(r))) > 0);
  return "";
}

// ------------------------------------------------------------------ CPU ranks as threads of one process
// ucclCommInitAll on the host backend: three communicators, one thread each, through the real
// bootstrap, proxy threads, FIFOs and the socket plugin.  Under ThreadSanitizer this is the race
// check of the whole host data path.
std::string testCpuRankThreads() {
  const char* prevBackend = getenv("UCCL_BACKEND");
  const std::string keep = prevBackend ? prevBackend : "";
  const char* prevIf = getenv("UCCL_BOOTSTRAP_IFNAME");
  const std::string keepIf = prevIf ? prevIf : "";
  setenv("UCCL_BACKEND", "cpu", 1);
  setenv("UCCL_BOOTSTRAP_IFNAME", "lo", 1);
  constexpr int n = 3;
  constexpr size_t count = 70001;  // not a multiple of anything
  ucclComm_t comms[n] = {};
  ucclResult_t rc = ucclCommInitAll(comms, n, nullptr);
  std::string fail;
  if (rc == ucclSuccess) {
    std::vector<std::vector<float>> buf(n, std::vector<float>(count));
    std::vector<std::vector<float>> gathered(n, std::vector<float>(count * n));
    for (int r = 0; r < n; ++r)
      for (size_t i = 0; i < count; ++i) buf[r][i] = static_cast<float>(r + 1) + static_cast<float>(i % 7);
    std::vector<ucclResult_t> res(n, ucclSuccess);
    std::vector<std::thread> th;
    for (int r = 0; r < n; ++r)
      th.emplace_back([&, r] {
        ucclResult_t e = ucclAllGather(buf[r].data(), gathered[r].data(), count, ucclFloat32, comms[r], nullptr);
        if (e == ucclSuccess) e = ucclAllReduce(buf[r].data(), buf[r].data(), count, ucclFloat32, ucclSum, comms[r], nullptr);
        res[r] = e;
      });
    for (auto& t : th) t.join();
    for (int r = 0; r < n && fail.empty(); ++r) {
      if (res[r] != ucclSuccess) fail = std::string("collective failed: ") + ucclGetErrorString(res[r]);
      for (size_t i = 0; i < count && fail.empty(); i += 997) {
        const float want = 6.f + 3.f * static_cast<float>(i % 7);
        if (buf[r][i] != want) fail = "wrong all-reduce value";
        for (int s = 0; s < n; ++s)
          if (gathered[r][s * count + i] != static_cast<float>(s + 1) + static_cast<float>(i % 7)) fail = "wrong all-gather value";
      }
    }
    for (int r = 0; r < n; ++r) ucclCommDestroy(comms[r]);
  } else {
    fail = std::string("ucclCommInitAll: ") + ucclGetErrorString(rc);
  }
  if (prevBackend) setenv("UCCL_BACKEND", keep.c_str(), 1); else unsetenv("UCCL_BACKEND");
  if (prevIf) setenv("UCCL_BOOTSTRAP_IFNAME", keepIf.c_str(), 1); else unsetenv("UCCL_BOOTSTRAP_IFNAME");
  return fail;
}

struct Case {
  const char* name;
  std::function<std::string()> fn;
};
const std::vector<Case>& cases() {
  static const std::vector<Case> all = {
      {"proxy_in_order", testProxyInOrder},
      {"proxy_immediate_completion", testProxyImmediateCompletion},
      {"proxy_busy_and_signal", testProxyBusyAndSignal},
      {"proxy_errors", testProxyErrors},
      {"ll128_codec", testLL128},
      {"ring_schedule", testRingSchedule},
      {"tuner", testTuner},
      {"plugin_loader", testPluginLoader},
      {"socket_loopback", testSocketLoopback},
      {"topology", testTopology},
      {"conversions", testConversions},
      {"config", testConfig},
      {"api_rules", testApiRules},
      {"cpu_rank_threads", testCpuRankThreads},
  };
  return all;
}

}  // namespace
}  // namespace uccl

extern "C" int ucclSelfTestCount(void) { return static_cast<int>(uccl::cases().size()); }
extern "C" const char* ucclSelfTestName(int index) {
  if (index < 0 || index >= ucclSelfTestCount()) return "";
  return uccl::cases()[index].name;
}
extern "C" int ucclSelfTestRun(const char* name, char* report, size_t reportLen) {
  if (report && reportLen) report[0] = 0;
  for (const auto& c : uccl::cases()) {
    if (strcmp(c.name, name) != 0) continue;
    std::string r = c.fn();
    if (report && reportLen) snprintf(report, reportLen, "%s", r.c_str());
    return r.empty() ? 0 : 1;
  }
  if (report && reportLen) snprintf(report, reportLen, "no such self test: %s", name);
  return 2;
}
