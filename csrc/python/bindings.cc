// pybind11 module `_uccl_bindings`: a thin shim over the C ABI in include/uccl.h.
// Device and host buffers cross the boundary as integer addresses (tensor.data_ptr()) and
// CUDA streams as integer handles (torch.cuda.current_stream().cuda_stream), which keeps the
// module free of any libtorch dependency -- the same convention as the reference's shim
// (bindings/python/uccl_bindings.cc:54-103), extended to the whole API.  Every call releases
// the GIL: communicator creation and the CPU backend block on other ranks.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "uccl.h"

namespace py = pybind11;

namespace {

struct UcclError : std::runtime_error {
  int code;
  UcclError(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

void check(ucclResult_t r, const char* what, ucclComm_t comm = nullptr) {
  if (r == ucclSuccess) return;
  std::string msg = std::string(what) + ": " + ucclGetErrorString(r);
  if (comm) {
    const char* last = ucclGetLastError(comm);
    if (last && *last) msg += std::string(" (") + last + ")";
  }
  throw UcclError(static_cast<int>(r), msg);
}

inline void* P(uintptr_t v) { return reinterpret_cast<void*>(v); }
inline ucclComm_t C(uintptr_t v) { return reinterpret_cast<ucclComm_t>(v); }
inline ucclDataType_t DT(int v) { return static_cast<ucclDataType_t>(v); }

ucclUniqueId idFromBytes(const py::bytes& b) {
  std::string s = b;
  if (s.size() != UCCL_UNIQUE_ID_BYTES) throw std::invalid_argument("unique id must be 128 bytes");
  ucclUniqueId id;
  std::memcpy(id.internal, s.data(), UCCL_UNIQUE_ID_BYTES);
  return id;
}

}  // namespace


PYBIND11_MODULE(_uccl_bindings, m) {
  m.doc() = "Python bindings of the sm_100a unified collective library";
  using nogil = py::call_guard<py::gil_scoped_release>;

  static py::exception<UcclError> exc(m, "UcclError", PyExc_RuntimeError);
  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const UcclError& e) {
      py::set_error(exc, e.what());
    }
  });

  m.attr("UNIQUE_ID_BYTES") = UCCL_UNIQUE_ID_BYTES;
  m.attr("MAX_RANKS") = UCCL_MAX_RANKS;

  m.def("get_version", [] {
    int v = 0;
    check(ucclGetVersion(&v), "ucclGetVersion");
    return v;
  });
  m.def("get_error_string", [](int code) { return std::string(ucclGetErrorString(static_cast<ucclResult_t>(code))); });

  // ---------------------------------------------------------------- lifecycle
  m.def("get_unique_id", [] {
    ucclUniqueId id;
    check(ucclGetUniqueId(&id), "ucclGetUniqueId");
    return py::bytes(id.internal, UCCL_UNIQUE_ID_BYTES);
  });
  m.def("unique_id_from_address", [](const std::string& ip, int port, uint64_t seed) {
    ucclUniqueId id;
    check(ucclUniqueIdFromAddress(ip.c_str(), port, seed, &id), "ucclUniqueIdFromAddress");
    return py::bytes(id.internal, UCCL_UNIQUE_ID_BYTES);
  });
  m.def("serve_unique_id", [](const py::bytes& b) {
    ucclUniqueId id = idFromBytes(b);
    check(ucclServeUniqueId(&id), "ucclServeUniqueId");
  });
  m.def("comm_init_rank",
        [](int nranks, const py::bytes& idb, int rank) {
          ucclUniqueId id = idFromBytes(idb);
          ucclComm_t comm = nullptr;
          ucclResult_t r;
          {
            py::gil_scoped_release rel;
            r = ucclCommInitRank(&comm, nranks, id, rank);
          }
          check(r, "ucclCommInitRank");
          return reinterpret_cast<uintptr_t>(comm);
        },
        py::arg("nranks"), py::arg("unique_id"), py::arg("rank"));
  m.def("comm_init_all", [](int ndev, const std::vector<int>& devlist) {
    std::vector<ucclComm_t> comms(ndev, nullptr);
    ucclResult_t r;
    {
      py::gil_scoped_release rel;
      r = ucclCommInitAll(comms.data(), ndev, devlist.empty() ? nullptr : devlist.data());
    }
    check(r, "ucclCommInitAll");
    std::vector<uintptr_t> out;
    for (ucclComm_t c : comms) out.push_back(reinterpret_cast<uintptr_t>(c));
    return out;
  });
  m.def("comm_finalize", [](uintptr_t c) { check(ucclCommFinalize(C(c)), "ucclCommFinalize", C(c)); }, nogil());
  m.def("comm_destroy", [](uintptr_t c) { check(ucclCommDestroy(C(c)), "ucclCommDestroy"); }, nogil());
  m.def("comm_abort", [](uintptr_t c) { check(ucclCommAbort(C(c)), "ucclCommAbort"); }, nogil());
  m.def("comm_count", [](uintptr_t c) {
    int n = 0;
    check(ucclCommCount(C(c), &n), "ucclCommCount");
    return n;
  });
  m.def("comm_rank", [](uintptr_t c) {
    int r = 0;
    check(ucclCommUserRank(C(c), &r), "ucclCommUserRank");
    return r;
  });
  m.def("get_last_error", [](uintptr_t c) { return std::string(ucclGetLastError(C(c))); });
  m.def("get_async_error", [](uintptr_t c) {
    ucclResult_t e = ucclSuccess;
    check(ucclCommGetAsyncError(C(c), &e), "ucclCommGetAsyncError");
    return static_cast<int>(e);
  });

  // ---------------------------------------------------------------- collectives
  m.def("allreduce",
        [](uintptr_t c, uintptr_t send, uintptr_t recv, size_t count, int dt, uintptr_t stream) {
          check(ucclAllReduce(P(send), P(recv), count, DT(dt), ucclSum, C(c), P(stream)), "ucclAllReduce", C(c));
        }, nogil());
  m.def("allreduce_ex", [](uintptr_t c, uintptr_t send, uintptr_t recv, size_t count, int inType, int outType, float scale,
                           uintptr_t scales, uintptr_t stream) {
    check(ucclAllReduceEx(P(send), P(recv), count, DT(inType), DT(outType), scale, static_cast<float*>(P(scales)), C(c), P(stream)),
          "ucclAllReduceEx", C(c));
  }, nogil());
  m.def("reduce_scatter_ex", [](uintptr_t c, uintptr_t send, uintptr_t recv, size_t recvcount, int inType, int outType,
                                float scale, uintptr_t scales, uintptr_t stream) {
    check(ucclReduceScatterEx(P(send), P(recv), recvcount, DT(inType), DT(outType), scale, static_cast<float*>(P(scales)), C(c),
                              P(stream)),
          "ucclReduceScatterEx", C(c));
  }, nogil());
  m.def("allgather",
        [](uintptr_t c, uintptr_t send, uintptr_t recv, size_t sendcount, int dt, uintptr_t stream) {
          check(ucclAllGather(P(send), P(recv), sendcount, DT(dt), C(c), P(stream)), "ucclAllGather", C(c));
        }, nogil());
  m.def("reduce_scatter",
        [](uintptr_t c, uintptr_t send, uintptr_t recv, size_t recvcount, int dt, uintptr_t stream) {
          check(ucclReduceScatter(P(send), P(recv), recvcount, DT(dt), ucclSum, C(c), P(stream)), "ucclReduceScatter", C(c));
        }, nogil());
  m.def("broadcast",
        [](uintptr_t c, uintptr_t send, uintptr_t recv, size_t count, int dt, int root, uintptr_t stream) {
          check(ucclBroadcast(P(send), P(recv), count, DT(dt), root, C(c), P(stream)), "ucclBroadcast", C(c));
        }, nogil());
  m.def("reduce",
        [](uintptr_t c, uintptr_t send, uintptr_t recv, size_t count, int dt, int root, uintptr_t stream) {
          check(ucclReduce(P(send), P(recv), count, DT(dt), ucclSum, root, C(c), P(stream)), "ucclReduce", C(c));
        }, nogil());
  m.def("alltoall",
        [](uintptr_t c, uintptr_t send, uintptr_t recv, size_t count, int dt, uintptr_t stream) {
          check(ucclAllToAll(P(send), P(recv), count, DT(dt), C(c), P(stream)), "ucclAllToAll", C(c));
        }, nogil());
  m.def("send",
        [](uintptr_t c, uintptr_t buf, size_t count, int dt, int peer, uintptr_t stream) {
          check(ucclSend(P(buf), count, DT(dt), peer, C(c), P(stream)), "ucclSend", C(c));
        }, nogil());
  m.def("recv",
        [](uintptr_t c, uintptr_t buf, size_t count, int dt, int peer, uintptr_t stream) {
          check(ucclRecv(P(buf), count, DT(dt), peer, C(c), P(stream)), "ucclRecv", C(c));
        }, nogil());
  m.def("group_start", [] { check(ucclGroupStart(), "ucclGroupStart"); });
  m.def("group_end", [] { check(ucclGroupEnd(), "ucclGroupEnd"); }, nogil());

  // ---------------------------------------------------------------- symmetric memory
  m.def("mem_alloc", [](uintptr_t c, size_t size) {
    void* p = nullptr;
    check(ucclMemAlloc(&p, size, C(c)), "ucclMemAlloc", C(c));
    return reinterpret_cast<uintptr_t>(p);
  }, nogil());
  m.def("mem_free", [](uintptr_t c, uintptr_t p) { check(ucclMemFree(P(p), C(c)), "ucclMemFree", C(c)); }, nogil());
  m.def("mem_check", [](uintptr_t c) { check(ucclMemCheck(C(c)), "ucclMemCheck", C(c)); }, nogil());
  m.def("mem_peer_pointer", [](uintptr_t c, uintptr_t p, int peer) {
    void* out = nullptr;
    check(ucclMemPeerPointer(P(p), peer, C(c), &out), "ucclMemPeerPointer", C(c));
    return reinterpret_cast<uintptr_t>(out);
  });
  m.def("mem_multicast_pointer", [](uintptr_t c, uintptr_t p) {
    void* out = nullptr;
    check(ucclMemMulticastPointer(P(p), C(c), &out), "ucclMemMulticastPointer", C(c));
    return reinterpret_cast<uintptr_t>(out);
  });

  // ---------------------------------------------------------------- introspection
  m.def("comm_info", [](uintptr_t c) {
    ucclCommInfo_t i;
    check(ucclCommGetInfo(C(c), &i), "ucclCommGetInfo");
    py::dict d;
    d["rank"] = i.rank; d["nranks"] = i.nranks; d["nnodes"] = i.nnodes;
    d["local_rank"] = i.localRank; d["local_ranks"] = i.localRanks; d["cuda_device"] = i.cudaDevice;
    d["n_channels"] = i.nChannels; d["nvls"] = i.nvlsSupported; d["p2p_mode"] = i.p2pMode;
    d["net_active"] = i.netActive; d["net_name"] = std::string(i.netName); d["staging_bytes"] = i.stagingBytes;
    return d;
  });
  m.def("comm_counters", [](uintptr_t c) {
    ucclCounters_t k;
    check(ucclCommGetCounters(C(c), &k), "ucclCommGetCounters");
    py::dict d;
    d["ops"] = std::vector<uint64_t>(k.ops, k.ops + 8);
    d["bytes"] = std::vector<uint64_t>(k.bytes, k.bytes + 8);
    d["algo_hist"] = std::vector<uint64_t>(k.algoHist, k.algoHist + ucclNumAlgos);
    d["proxy_posts"] = k.proxyPosts; d["proxy_completions"] = k.proxyCompletions;
    d["proxy_heartbeat"] = k.proxyHeartbeat; d["wait_timeouts"] = k.waitTimeouts;
    return d;
  });
  m.def("query_tuning", [](uintptr_t c, int coll, size_t bytes, bool symmetric) {
    ucclAlgo_t a; ucclProto_t p; int n = 0;
    check(ucclCommQueryTuning(C(c), static_cast<ucclCollKind_t>(coll), bytes, symmetric ? 1 : 0, &a, &p, &n), "ucclCommQueryTuning");
    return py::make_tuple(static_cast<int>(a), static_cast<int>(p), n);
  });
  m.def("load_tuning", [](uintptr_t c, const std::string& path) { check(ucclCommLoadTuning(C(c), path.c_str()), "ucclCommLoadTuning", C(c)); });
  m.def("set_algo", [](uintptr_t c, int algo, int proto) {
    check(ucclCommSetAlgo(C(c), static_cast<ucclAlgo_t>(algo), static_cast<ucclProto_t>(proto)), "ucclCommSetAlgo");
  });

  m.def("set_blocks", [](uintptr_t c, int blocks) { check(ucclCommSetBlocks(C(c), blocks), "ucclCommSetBlocks"); });
  m.def("set_fused_norm_rows", [](uintptr_t c, int rows) { check(ucclCommSetFusedNormRows(C(c), rows), "ucclCommSetFusedNormRows"); });
  m.def("set_fused_rs_reducers", [](uintptr_t c, int n) { check(ucclCommSetFusedRsReducers(C(c), n), "ucclCommSetFusedRsReducers"); });
  m.def("set_fused_options", [](uintptr_t c, int agMode, int commCtas, int ceChunks) {
    check(ucclCommSetFusedOptions(C(c), agMode, commCtas, ceChunks), "ucclCommSetFusedOptions");
  });

  // ---------------------------------------------------------------- local ops
  m.def("gemm_bf16",
        [](uintptr_t A, uintptr_t B, uintptr_t Cp, int M, int N, int K, int lda, int ldb, int ldc, int epilogue,
           uintptr_t stream) {
          check(ucclGemmBf16(P(A), P(B), P(Cp), M, N, K, lda, ldb, ldc, epilogue, P(stream)), "ucclGemmBf16");
        },
        py::arg("A"), py::arg("B"), py::arg("C"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("lda"),
        py::arg("ldb"), py::arg("ldc"), py::arg("epilogue") = 0, py::arg("stream") = 0);

  // ---------------------------------------------------------------- fused kernels
  m.def("allreduce_residual_rmsnorm",
        [](uintptr_t c, uintptr_t x, uintptr_t residual, uintptr_t gamma, uintptr_t out, uintptr_t residualOut, int tokens,
           int hidden, float eps, uintptr_t stream) {
          check(ucclAllReduceResidualRMSNorm(P(x), P(residual), P(gamma), P(out), P(residualOut), tokens, hidden, eps, C(c),
                                             P(stream)),
                "ucclAllReduceResidualRMSNorm", C(c));
        }, nogil());
  m.def("allgather_gemm",
        [](uintptr_t c, uintptr_t xShard, uintptr_t xFull, uintptr_t W, uintptr_t out, int M, int N, int K, int epilogue,
           uintptr_t stream) {
          check(ucclAllGatherGemm(P(xShard), P(xFull), P(W), P(out), M, N, K, epilogue, C(c), P(stream)), "ucclAllGatherGemm", C(c));
        }, nogil());
  m.def("gemm_reduce_scatter",
        [](uintptr_t c, uintptr_t A, uintptr_t W, uintptr_t cPartial, uintptr_t out, int M, int N, int K, uintptr_t stream) {
          check(ucclGemmReduceScatter(P(A), P(W), P(cPartial), P(out), M, N, K, C(c), P(stream)), "ucclGemmReduceScatter", C(c));
        }, nogil());

  // ---------------------------------------------------------------- MoE dispatch / combine
  m.def("moe_create", [](uintptr_t c, int maxTokens, int hidden, int experts, int topk, float factor) {
    ucclMoeContext_t ctx = nullptr;
    check(ucclMoeCreate(&ctx, maxTokens, hidden, experts, topk, factor, C(c)), "ucclMoeCreate", C(c));
    return reinterpret_cast<uintptr_t>(ctx);
  }, nogil());
  m.def("moe_destroy", [](uintptr_t ctx) { check(ucclMoeDestroy(reinterpret_cast<ucclMoeContext_t>(ctx)), "ucclMoeDestroy"); }, nogil());
  m.def("moe_layout", [](uintptr_t ctx) {
    ucclMoeLayout_t l;
    check(ucclMoeGetLayout(reinterpret_cast<ucclMoeContext_t>(ctx), &l), "ucclMoeGetLayout");
    py::dict d;
    d["recv_x"] = reinterpret_cast<uintptr_t>(l.recvX);
    d["recv_scale"] = reinterpret_cast<uintptr_t>(l.recvScale);
    d["recv_meta"] = reinterpret_cast<uintptr_t>(l.recvMeta);
    d["recv_counts"] = reinterpret_cast<uintptr_t>(l.recvCounts);
    d["expert_out"] = reinterpret_cast<uintptr_t>(l.expertOut);
    d["rows_per_source"] = l.rowsPerSource;
    d["nranks"] = l.nranks;
    return d;
  });
  m.def("moe_dispatch", [](uintptr_t ctx, uintptr_t x, uintptr_t idx, int tokens, uintptr_t stream) {
    check(ucclMoeDispatch(reinterpret_cast<ucclMoeContext_t>(ctx), P(x), static_cast<const int32_t*>(P(idx)), tokens, P(stream)),
          "ucclMoeDispatch");
  }, nogil());
  m.def("moe_combine", [](uintptr_t ctx, uintptr_t w, int tokens, uintptr_t out, uintptr_t stream) {
    check(ucclMoeCombine(reinterpret_cast<ucclMoeContext_t>(ctx), static_cast<const float*>(P(w)), tokens, P(out), P(stream)),
          "ucclMoeCombine");
  }, nogil());
  m.def("moe_overflow", [](uintptr_t ctx) {
    unsigned int rows = 0;
    check(ucclMoeOverflow(reinterpret_cast<ucclMoeContext_t>(ctx), &rows), "ucclMoeOverflow");
    return rows;
  });

  // ---------------------------------------------------------------- one-sided windows
  m.def("window_register", [](uintptr_t c, uintptr_t buf, size_t size) {
    ucclWindow_t w = nullptr;
    check(ucclCommWindowRegister(&w, P(buf), size, C(c)), "ucclCommWindowRegister", C(c));
    return reinterpret_cast<uintptr_t>(w);
  }, nogil());
  m.def("window_deregister", [](uintptr_t w) {
    check(ucclCommWindowDeregister(reinterpret_cast<ucclWindow_t>(w)), "ucclCommWindowDeregister");
  }, nogil());
  m.def("put", [](uintptr_t c, uintptr_t local, size_t count, int dt, int peer, uintptr_t win, size_t off, uintptr_t stream) {
    check(ucclPut(P(local), count, DT(dt), peer, reinterpret_cast<ucclWindow_t>(win), off, C(c), P(stream)), "ucclPut", C(c));
  }, nogil());
  m.def("get", [](uintptr_t c, uintptr_t local, size_t count, int dt, int peer, uintptr_t win, size_t off, uintptr_t stream) {
    check(ucclGet(P(local), count, DT(dt), peer, reinterpret_cast<ucclWindow_t>(win), off, C(c), P(stream)), "ucclGet", C(c));
  }, nogil());
  m.def("put_signal", [](uintptr_t c, uintptr_t local, size_t count, int dt, int peer, uintptr_t win, size_t off, uintptr_t stream) {
    check(ucclPutSignal(P(local), count, DT(dt), peer, reinterpret_cast<ucclWindow_t>(win), off, 0, 0, 0, C(c), P(stream)),
          "ucclPutSignal", C(c));
  }, nogil());
  m.def("get_signal", [](uintptr_t c, uintptr_t local, size_t count, int dt, int peer, uintptr_t win, size_t off, uintptr_t stream) {
    check(ucclGetSignal(P(local), count, DT(dt), peer, reinterpret_cast<ucclWindow_t>(win), off, 0, 0, 0, C(c), P(stream)),
          "ucclGetSignal", C(c));
  }, nogil());
  m.def("signal", [](uintptr_t c, int peer, uintptr_t stream) {
    check(ucclSignal(peer, 0, 0, 0, C(c), P(stream)), "ucclSignal", C(c));
  }, nogil());
  m.def("wait_signal", [](uintptr_t c, uintptr_t win, const std::vector<int>& peers, const std::vector<int>& counts, uintptr_t stream) {
    if (peers.size() != counts.size() || peers.size() > 8) throw std::invalid_argument("need 1..8 (peer, count) pairs");
    ucclWaitSignalDesc_t d[8];
    for (size_t i = 0; i < peers.size(); ++i) d[i] = {counts[i], peers[i], 0, 0, reinterpret_cast<ucclWindow_t>(win)};
    check(ucclWaitSignal(static_cast<int>(peers.size()), d, C(c), P(stream)), "ucclWaitSignal", C(c));
  }, nogil());

}
