#include "cuda_driver.h"

#include <mutex>

namespace uccl {

namespace {
template <typename Fn>
bool resolve(const char* name, Fn* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
    (void)cudaGetLastError();
    *out = nullptr;
    return false;
  }
  *out = reinterpret_cast<Fn>(fn);
  return true;
}
}  // namespace

const DriverApi& driverApi() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
      (void)cudaGetLastError();
      return;
    }
    bool ok = true;
    ok &= resolve("cuTensorMapEncodeTiled", &api.tensorMapEncodeTiled);
    ok &= resolve("cuMemCreate", &api.memCreate);
    ok &= resolve("cuMemRelease", &api.memRelease);
    ok &= resolve("cuMemAddressReserve", &api.memAddressReserve);
    ok &= resolve("cuMemAddressFree", &api.memAddressFree);
    ok &= resolve("cuMemMap", &api.memMap);
    ok &= resolve("cuMemUnmap", &api.memUnmap);
    ok &= resolve("cuMemSetAccess", &api.memSetAccess);
    ok &= resolve("cuMemExportToShareableHandle", &api.memExportToShareableHandle);
    ok &= resolve("cuMemImportFromShareableHandle", &api.memImportFromShareableHandle);
    ok &= resolve("cuMemGetAllocationGranularity", &api.memGetAllocationGranularity);
    ok &= resolve("cuDeviceGetAttribute", &api.deviceGetAttribute);
    ok &= resolve("cuDeviceGet", &api.deviceGet);
    ok &= resolve("cuGetErrorString", &api.getErrorString);
    ok &= resolve("cuCtxGetCurrent", &api.ctxGetCurrent);
    ok &= resolve("cuMemGetAddressRange", &api.memGetAddressRange);
    // Multicast objects are optional (absent on drivers/GPUs without NVLS).
    resolve("cuMulticastCreate", &api.multicastCreate);
    resolve("cuMulticastAddDevice", &api.multicastAddDevice);
    resolve("cuMulticastBindMem", &api.multicastBindMem);
    resolve("cuMulticastUnbind", &api.multicastUnbind);
    resolve("cuMulticastGetGranularity", &api.multicastGetGranularity);
    api.ok = ok;
  });
  return api;
}

const char* driverErrorString(CUresult r) {
  const DriverApi& d = driverApi();
  const char* s = nullptr;
  if (d.getErrorString && d.getErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "unknown CUDA driver error";
}

}  // namespace uccl
