#include "host_coll.h"

#include <sched.h>
#include <string.h>

#include <algorithm>

#include "../core/log.h"
#include "ring_schedule.h"

namespace uccl {

// ------------------------------------------------------------------ scalar conversions
float bf16ToFloat(uint16_t v) {
  uint32_t u = static_cast<uint32_t>(v) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t floatToBf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest even
  return static_cast<uint16_t>(u >> 16);
}
float halfToFloat(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1f;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {  // subnormal
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      man &= 0x3ffu;
      u = sign | ((127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t floatToHalf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const int32_t exp = static_cast<int32_t>((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (((u >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t h = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return static_cast<uint16_t>(sign | h);
  }
  uint32_t h = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return static_cast<uint16_t>(sign | h);
}

void hostReduceInto(void* dst, const void* src, size_t count, ucclDataType_t dt) {
  switch (dt) {
    case ucclFloat32: {
      float* d = static_cast<float*>(dst);
      const float* s = static_cast<const float*>(src);
      for (size_t i = 0; i < count; ++i) d[i] += s[i];
      break;
    }
    case ucclBfloat16: {
      uint16_t* d = static_cast<uint16_t*>(dst);
      const uint16_t* s = static_cast<const uint16_t*>(src);
      for (size_t i = 0; i < count; ++i) d[i] = floatToBf16(bf16ToFloat(d[i]) + bf16ToFloat(s[i]));
      break;
    }
    case ucclFloat16: {
      uint16_t* d = static_cast<uint16_t*>(dst);
      const uint16_t* s = static_cast<const uint16_t*>(src);
      for (size_t i = 0; i < count; ++i) d[i] = floatToHalf(halfToFloat(d[i]) + halfToFloat(s[i]));
      break;
    }
    default:
      break;  // not reducible; callers reject these types earlier
  }
}

// ------------------------------------------------------------------ transfer engine
static bool connError(Comm* comm, NetConn* c, ucclResult_t* out) {
  const uint64_t err = __atomic_load_n(&c->fifo->error, __ATOMIC_ACQUIRE);
  if (err) {
    *out = static_cast<ucclResult_t>(err);
    return true;
  }
  if (comm->abortFlag.load(std::memory_order_relaxed)) {
    *out = ucclRemoteError;
    return true;
  }
  return false;
}

ucclResult_t hostRunXfers(Comm* comm, std::vector<HostXfer>& xfers) {
  size_t remaining = 0;
  for (HostXfer& x : xfers) {
    if (x.len == 0) continue;
    if (x.conns.empty()) return ucclInternalError;
    x.posted = x.done = 0;
    x.steps.clear();
    // a GPU kernel may have been the producer on these connections since the last host-driven
    // transfer: the FIFO tail is the single source of truth for the next step number
    for (NetConn* c : x.conns) c->step = fifoLoadAcquire(&c->fifo->tail);
    ++remaining;
  }
  uint64_t lastProgress = nowMs();
  uint32_t idle = 0;
  while (remaining) {
    bool moved = false;
    jitterPause(comm->cfg.jitterUs);
    for (HostXfer& x : xfers) {
      if (x.len == 0) continue;
      const size_t slot = x.conns[0]->slotBytes;
      const size_t nsub = (x.len + slot - 1) / slot;
      if (x.done == nsub) continue;
      ucclResult_t err;
      // post as many sub-chunks as the FIFOs take
      while (x.posted < nsub) {
        // a receive slot (and its FIFO entry) may only be re-posted after this thread consumed
        // what it held: never keep more than UCCL_STEPS unconsumed receives per connection
        if (!x.isSend && x.posted - x.done >= UCCL_STEPS * x.conns.size()) break;
        NetConn* c = x.conns[x.posted % x.conns.size()];
        if (connError(comm, c, &err)) return err;
        const uint64_t head = fifoLoadAcquire(&c->fifo->head);
        if (c->step - head >= UCCL_STEPS) break;  // no free slot on that connection yet
        const size_t off = x.posted * slot;
        const size_t n = std::min(slot, x.len - off);
        uint64_t step = 0;
        if (x.isSend) memcpy(netSlot(c, c->step), x.src + off, n);
        ucclResult_t r = netHostPost(comm, c, x.isSend ? FIFO_SEND : FIFO_RECV, n, &step);
        if (r != ucclSuccess) return r;
        x.steps.push_back(step);
        ++x.posted;
        moved = true;
      }
      // retire completed sub-chunks in order
      while (x.done < x.posted) {
        NetConn* c = x.conns[x.done % x.conns.size()];
        if (connError(comm, c, &err)) return err;
        const uint64_t step = x.steps[x.done];
        if (fifoLoadAcquire(&c->fifo->head) <= step) break;
        if (!x.isSend) {
          const size_t off = x.done * slot;
          const size_t n = std::min(slot, x.len - off);
          const size_t got = static_cast<size_t>(c->fifo->entries[step % UCCL_STEPS].result);
          if (got != n) {
            commSetError(comm, "short network message from rank %d: %zu of %zu bytes", c->peer, got, n);
            return ucclRemoteError;
          }
          const char* in = netSlot(c, step);
          if (x.reduce) hostReduceInto(x.dst + off, in, n / dataTypeSize(x.dtype), x.dtype);
          else memcpy(x.dst + off, in, n);
        }
        ++x.done;
        moved = true;
        if (x.done == nsub) --remaining;
      }
    }
    if (moved) {
      lastProgress = nowMs();
      idle = 0;
    } else if ((++idle & 0x3f) == 0) {
      if (nowMs() - lastProgress > comm->cfg.waitTimeoutMs) {
        commSetError(comm, "network transfer made no progress for %llu ms",
                     (unsigned long long)comm->cfg.waitTimeoutMs);
        {
          std::lock_guard<std::mutex> lk(comm->ctrMu);
          comm->counters.waitTimeouts++;
        }
        commSetAsyncError(comm, ucclRemoteError);
        return ucclRemoteError;
      }
      sched_yield();
    }
  }
  return ucclSuccess;
}

namespace {

std::vector<NetConn*> ringSendConns(Comm* c) {
  std::vector<NetConn*> v;
  for (Channel& ch : c->channels)
    if (ch.netReady) v.push_back(&ch.send);
  return v;
}
std::vector<NetConn*> ringRecvConns(Comm* c) {
  std::vector<NetConn*> v;
  for (Channel& ch : c->channels)
    if (ch.netReady) v.push_back(&ch.recv);
  return v;
}

// Ring geometry: `pos` is this rank's position in the ring order, rankAt(p) the rank at position p.
int ringPos(Comm* c) { return c->channels[0].index; }
int rankAt(Comm* c, int position) {
  const int n = c->nRanks, pos = c->channels[0].index;
  return c->channels[0].userRanks[((position - pos) % n + n) % n];
}

ucclResult_t ringStep(Comm* c, const char* src, size_t sendLen, char* dst, size_t recvLen, bool reduce,
                      ucclDataType_t dt) {
  std::vector<HostXfer> xs(2);
  xs[0].conns = ringSendConns(c);
  xs[0].isSend = true;
  xs[0].src = src;
  xs[0].len = sendLen;
  xs[1].conns = ringRecvConns(c);
  xs[1].isSend = false;
  xs[1].dst = dst;
  xs[1].len = recvLen;
  xs[1].reduce = reduce;
  xs[1].dtype = dt;
  if (xs[0].conns.empty() || xs[1].conns.empty()) {
    commSetError(c, "network ring is not connected");
    return ucclInternalError;
  }
  return hostRunXfers(c, xs);
}

}  // namespace

ucclResult_t hostAllReduce(Comm* c, const void* send, void* recv, size_t count, ucclDataType_t dt) {
  const size_t es = dataTypeSize(dt);
  if (send != recv) memmove(recv, send, count * es);
  const int n = c->nRanks;
  if (n == 1) return ucclSuccess;
  const int r = ringPos(c);  // chunks are labelled by ring position; the result is symmetric
  char* buf = static_cast<char*>(recv);
  // reduce-scatter phase
  for (int s = 0; s < n - 1; ++s) {
    const int sc = ringRsSendChunk(r, s, n), rc = ringRsRecvChunk(r, s, n);
    size_t so, sl, ro, rl;
    ringChunk(count, n, sc, &so, &sl);
    ringChunk(count, n, rc, &ro, &rl);
    ucclResult_t e = ringStep(c, buf + so * es, sl * es, buf + ro * es, rl * es, true, dt);
    if (e != ucclSuccess) return e;
  }
  // all-gather phase
  for (int s = 0; s < n - 1; ++s) {
    const int sc = ringAgSendChunk(r, s, n), rc = ringAgRecvChunk(r, s, n);
    size_t so, sl, ro, rl;
    ringChunk(count, n, sc, &so, &sl);
    ringChunk(count, n, rc, &ro, &rl);
    ucclResult_t e = ringStep(c, buf + so * es, sl * es, buf + ro * es, rl * es, false, dt);
    if (e != ucclSuccess) return e;
  }
  return ucclSuccess;
}

ucclResult_t hostAllGather(Comm* c, const void* send, void* recv, size_t sendcount, ucclDataType_t dt) {
  const size_t bytes = sendcount * dataTypeSize(dt);
  const int n = c->nRanks, r = c->rank;
  char* out = static_cast<char*>(recv);
  if (out + static_cast<size_t>(r) * bytes != send) memmove(out + static_cast<size_t>(r) * bytes, send, bytes);
  const int pos = n > 1 ? ringPos(c) : 0;
  for (int s = 0; s < n - 1; ++s) {
    const int sc = rankAt(c, pos - s), rc = rankAt(c, pos - s - 1);
    ucclResult_t e = ringStep(c, out + static_cast<size_t>(sc) * bytes, bytes, out + static_cast<size_t>(rc) * bytes,
                              bytes, false, dt);
    if (e != ucclSuccess) return e;
  }
  return ucclSuccess;
}

ucclResult_t hostReduceScatter(Comm* c, const void* send, void* recv, size_t recvcount, ucclDataType_t dt) {
  const size_t es = dataTypeSize(dt), bytes = recvcount * es;
  const int n = c->nRanks, r = c->rank;
  if (n == 1) {
    if (send != recv) memmove(recv, send, bytes);
    return ucclSuccess;
  }
  std::vector<char> work(static_cast<size_t>(n) * bytes);
  memcpy(work.data(), send, work.size());
  const int pos = ringPos(c);
  for (int s = 0; s < n - 1; ++s) {
    const int sc = rankAt(c, pos - s - 1), rc = rankAt(c, pos - s - 2);
    ucclResult_t e = ringStep(c, work.data() + static_cast<size_t>(sc) * bytes, bytes,
                              work.data() + static_cast<size_t>(rc) * bytes, bytes, true, dt);
    if (e != ucclSuccess) return e;
  }
  memcpy(recv, work.data() + static_cast<size_t>(r) * bytes, bytes);
  return ucclSuccess;
}

ucclResult_t hostBroadcast(Comm* c, const void* send, void* recv, size_t count, ucclDataType_t dt, int root) {
  const size_t bytes = count * dataTypeSize(dt);
  const int n = c->nRanks, r = c->rank;
  if (r == root && send != recv) memmove(recv, send, bytes);
  if (n == 1) return ucclSuccess;
  const int next = c->channels[0].next;
  // pipeline along the ring: receive a piece from the predecessor, pass it on unless the
  // successor is the root.  Pieces are bounded so that forwarding overlaps receiving.
  const size_t piece = c->channels[0].send.slotBytes * UCCL_STEPS;
  char* buf = static_cast<char*>(recv);
  for (size_t off = 0; off < bytes || off == 0; off += piece) {
    const size_t nb = std::min(piece, bytes - off);
    if (r != root) {
      ucclResult_t e = ringStep(c, nullptr, 0, buf + off, nb, false, dt);
      if (e != ucclSuccess) return e;
    }
    if (next != root) {
      ucclResult_t e = ringStep(c, buf + off, nb, nullptr, 0, false, dt);
      if (e != ucclSuccess) return e;
    }
    if (bytes == 0) break;
  }
  return ucclSuccess;
}

ucclResult_t hostReduce(Comm* c, const void* send, void* recv, size_t count, ucclDataType_t dt, int root) {
  const size_t es = dataTypeSize(dt), bytes = count * es;
  const int n = c->nRanks, r = c->rank;
  if (n == 1) {
    if (send != recv) memmove(recv, send, bytes);
    return ucclSuccess;
  }
  // chain root+1 -> root+2 -> ... -> root; every hop adds its own contribution
  const bool isFirst = c->channels[0].prev == root;
  std::vector<char> tmp;
  char* acc;
  if (r == root) {
    if (send != recv) memmove(recv, send, bytes);
    acc = static_cast<char*>(recv);
  } else {
    tmp.assign(static_cast<const char*>(send), static_cast<const char*>(send) + bytes);
    acc = tmp.data();
  }
  if (!isFirst) {
    ucclResult_t e = ringStep(c, nullptr, 0, acc, bytes, true, dt);
    if (e != ucclSuccess) return e;
  }
  if (r != root) {
    ucclResult_t e = ringStep(c, acc, bytes, nullptr, 0, false, dt);
    if (e != ucclSuccess) return e;
  }
  return ucclSuccess;
}

ucclResult_t hostAllToAll(Comm* c, const void* send, void* recv, size_t count, ucclDataType_t dt) {
  const size_t bytes = count * dataTypeSize(dt);
  const int n = c->nRanks, r = c->rank;
  const char* in = static_cast<const char*>(send);
  char* out = static_cast<char*>(recv);
  memmove(out + static_cast<size_t>(r) * bytes, in + static_cast<size_t>(r) * bytes, bytes);
  if (n == 1) return ucclSuccess;
  std::vector<int> peers;
  for (int p = 0; p < n; ++p)
    if (p != r) peers.push_back(p);
  ucclResult_t e = netEnsurePeers(c, peers);
  if (e != ucclSuccess) return e;
  std::vector<HostXfer> xs;
  for (int p : peers) {
    HostXfer s;
    s.conns = {c->meshSend[p].get()};
    s.isSend = true;
    s.src = in + static_cast<size_t>(p) * bytes;
    s.len = bytes;
    xs.push_back(s);
    HostXfer rv;
    rv.conns = {c->meshRecv[p].get()};
    rv.isSend = false;
    rv.dst = out + static_cast<size_t>(p) * bytes;
    rv.len = bytes;
    xs.push_back(rv);
  }
  return hostRunXfers(c, xs);
}

ucclResult_t hostSendRecv(Comm* c, const std::vector<HostP2pOp>& ops) {
  std::vector<int> peers;
  for (const HostP2pOp& op : ops)
    if (op.peer != c->rank) peers.push_back(op.peer);
  std::sort(peers.begin(), peers.end());
  peers.erase(std::unique(peers.begin(), peers.end()), peers.end());
  if (!peers.empty()) {
    ucclResult_t e = netEnsurePeers(c, peers);
    if (e != ucclSuccess) return e;
  }
  // Operations on one connection run back to back in posting order; different connections
  // progress concurrently, which is what makes grouped send+recv pairs deadlock-free.
  std::vector<size_t> order(ops.size());
  for (size_t i = 0; i < ops.size(); ++i) order[i] = i;
  std::vector<bool> done(ops.size(), false);
  // self send/recv pairs are matched locally
  for (size_t i = 0; i < ops.size(); ++i) {
    if (done[i] || ops[i].peer != c->rank || !ops[i].isSend) continue;
    for (size_t j = 0; j < ops.size(); ++j)
      if (!done[j] && ops[j].peer == c->rank && !ops[j].isSend && ops[j].bytes == ops[i].bytes) {
        memmove(ops[j].recv, ops[i].send, ops[i].bytes);
        done[i] = done[j] = true;
        break;
      }
    if (!done[i]) {
      commSetError(c, "send to self without a matching recv in the same group");
      return ucclInvalidUsage;
    }
  }
  while (true) {
    std::vector<HostXfer> xs;
    std::vector<size_t> picked;
    std::vector<NetConn*> busy;
    for (size_t i = 0; i < ops.size(); ++i) {
      if (done[i]) continue;
      const HostP2pOp& op = ops[i];
      if (op.peer == c->rank) {
        commSetError(c, "recv from self without a matching send in the same group");
        return ucclInvalidUsage;
      }
      NetConn* conn = op.isSend ? c->meshSend[op.peer].get() : c->meshRecv[op.peer].get();
      if (std::find(busy.begin(), busy.end(), conn) != busy.end()) continue;  // next round
      busy.push_back(conn);
      HostXfer x;
      x.conns = {conn};
      x.isSend = op.isSend;
      x.src = static_cast<const char*>(op.send);
      x.dst = static_cast<char*>(op.recv);
      x.len = op.bytes;
      xs.push_back(x);
      picked.push_back(i);
    }
    if (picked.empty()) break;
    ucclResult_t e = hostRunXfers(c, xs);
    if (e != ucclSuccess) return e;
    for (size_t i : picked) done[i] = true;
  }
  return ucclSuccess;
}

}  // namespace uccl
