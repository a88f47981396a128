// Per-operation tracing: an NVTX range around every enqueue, and -- when UCCL_TRACE_FILE is set --
// a pair of CUDA events around the launches of the operation, turned into one JSON line per
// operation ({"op", "bytes", "algo", "us"}) in <file>.<rank> when the communicator is destroyed.
// The reference has neither timers nor ranges, only TRACE log lines on API entry
// (src/collectives.cc:65,90,120).
#pragma once
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include "comm.h"

namespace uccl {

constexpr size_t kMaxTraceEvents = 8192;

class TraceScope {
 public:
  TraceScope(Comm* c, const char* name, size_t bytes, cudaStream_t stream) : c_(c), stream_(stream) {
    nvtxRangePushA(name);
    if (c->cfg.traceFile.empty() || c->trace.size() >= kMaxTraceEvents) return;
    TraceEvent ev{name, bytes, 0, nullptr, nullptr};
    if (cudaEventCreate(&ev.start) != cudaSuccess || cudaEventCreate(&ev.stop) != cudaSuccess) return;
    cudaEventRecord(ev.start, stream);
    c->trace.push_back(ev);
    active_ = true;
  }
  void setAlgo(int algo) {
    if (active_) c_->trace.back().algo = algo;
  }
  ~TraceScope() {
    if (active_) cudaEventRecord(c_->trace.back().stop, stream_);
    nvtxRangePop();
  }

 private:
  Comm* c_;
  cudaStream_t stream_;
  bool active_ = false;
};

// Writes the collected events and releases them (called once, from communicator teardown).
void traceDump(Comm* c);

}  // namespace uccl
