// Group semantics.  In the reference ucclGroupStart/End only count nesting depth and nothing is
// deferred (src/group.cc:20-50).  Here operations issued inside a group are queued per thread and
// run when the outermost ucclGroupEnd is reached; all point-to-point operations of one
// communicator in the group are fused into a single launch, which is what makes
// "send to next + recv from prev" safe to write in any order.
#include <map>
#include <vector>

#include "enqueue.h"
#include "log.h"

namespace uccl {

namespace {
thread_local int t_depth = 0;
thread_local std::vector<CollOp> t_queue;
}  // namespace

bool groupActive() { return t_depth > 0; }

ucclResult_t groupAppend(const CollOp& op) {
  t_queue.push_back(op);
  return ucclSuccess;
}

static ucclResult_t flushGroup() {
  std::vector<CollOp> q;
  q.swap(t_queue);
  ucclResult_t first = ucclSuccess;
  // point-to-point operations: one batch per communicator, in issue order
  std::vector<Comm*> order;
  std::map<Comm*, std::vector<CollOp>> p2p;
  for (const CollOp& op : q) {
    if (op.kind != ucclCollSendRecv) continue;
    if (!p2p.count(op.comm)) order.push_back(op.comm);
    p2p[op.comm].push_back(op);
  }
  for (const CollOp& op : q) {
    if (op.kind == ucclCollSendRecv) continue;
    ucclResult_t r = executeOp(op);
    if (r != ucclSuccess && first == ucclSuccess) first = r;
  }
  for (Comm* c : order) {
    ucclResult_t r = executeP2pBatch(c, p2p[c]);
    if (r != ucclSuccess && first == ucclSuccess) first = r;
  }
  return first;
}

}  // namespace uccl

extern "C" ucclResult_t ucclGroupStart(void) {
  ++uccl::t_depth;
  UCCL_LOG(TRACE, "ucclGroupStart depth=%d", uccl::t_depth);
  return ucclSuccess;
}

extern "C" ucclResult_t ucclGroupEnd(void) {
  if (uccl::t_depth <= 0) {
    UCCL_LOG(WARN, "ucclGroupEnd without a matching ucclGroupStart");
    return ucclInvalidUsage;
  }
  --uccl::t_depth;
  UCCL_LOG(TRACE, "ucclGroupEnd depth=%d queued=%zu", uccl::t_depth, uccl::t_queue.size());
  if (uccl::t_depth > 0) return ucclSuccess;
  return uccl::flushGroup();
}
