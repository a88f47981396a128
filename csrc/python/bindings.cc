// pybind11 module `_uccl_bindings`: a thin shim over the C ABI in include/uccl.h.
// Device and host buffers cross the boundary as integer addresses (tensor.data_ptr()) and
// CUDA streams as integer handles (torch.cuda.current_stream().cuda_stream), which keeps the
// module free of any libtorch dependency -- the same convention as the reference's shim
// (bindings/python/uccl_bindings.cc:54-103), extended to the whole API.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>

#include "uccl.h"

namespace py = pybind11;

namespace {

void check(ucclResult_t r, const char* what) {
  if (r != ucclSuccess) {
    throw std::runtime_error(std::string(what) + ": " + ucclGetErrorString(r));
  }
}

inline void* P(uintptr_t v) { return reinterpret_cast<void*>(v); }

}  // namespace


PYBIND11_MODULE(_uccl_bindings, m) {
  m.doc() = "Python bindings of the sm_100a unified collective library";

  m.def("get_version", [] {
    int v = 0;
    check(ucclGetVersion(&v), "ucclGetVersion");
    return v;
  });
  m.def("get_error_string", [](int code) { return std::string(ucclGetErrorString(static_cast<ucclResult_t>(code))); });

  m.def("gemm_bf16",
        [](uintptr_t A, uintptr_t B, uintptr_t C, int M, int N, int K, int lda, int ldb, int ldc, int epilogue,
           uintptr_t stream) {
          check(ucclGemmBf16(P(A), P(B), P(C), M, N, K, lda, ldb, ldc, epilogue, P(stream)), "ucclGemmBf16");
        },
        py::arg("A"), py::arg("B"), py::arg("C"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("lda"),
        py::arg("ldb"), py::arg("ldc"), py::arg("epilogue") = 0, py::arg("stream") = 0);

}
