// Lazily resolved CUDA driver entry points. The library links only against the CUDA runtime;
// driver symbols (VMM, multicast objects, tensor maps, stream memory operations) are looked up
// through cudaGetDriverEntryPoint so that the shared object still loads, and the CPU-rank
// backend still runs, on a machine that has no NVIDIA driver installed.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace uccl {

struct DriverApi {
  bool ok = false;
  decltype(&cuTensorMapEncodeTiled) tensorMapEncodeTiled = nullptr;
  decltype(&cuMemCreate) memCreate = nullptr;
  decltype(&cuMemRelease) memRelease = nullptr;
  decltype(&cuMemAddressReserve) memAddressReserve = nullptr;
  decltype(&cuMemAddressFree) memAddressFree = nullptr;
  decltype(&cuMemMap) memMap = nullptr;
  decltype(&cuMemUnmap) memUnmap = nullptr;
  decltype(&cuMemSetAccess) memSetAccess = nullptr;
  decltype(&cuMemExportToShareableHandle) memExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) memImportFromShareableHandle = nullptr;
  decltype(&cuMemGetAllocationGranularity) memGetAllocationGranularity = nullptr;
  decltype(&cuMulticastCreate) multicastCreate = nullptr;
  decltype(&cuMulticastAddDevice) multicastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) multicastBindMem = nullptr;
  decltype(&cuMulticastUnbind) multicastUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) multicastGetGranularity = nullptr;
  decltype(&cuDeviceGetAttribute) deviceGetAttribute = nullptr;
  decltype(&cuDeviceGet) deviceGet = nullptr;
  decltype(&cuGetErrorString) getErrorString = nullptr;
  decltype(&cuCtxGetCurrent) ctxGetCurrent = nullptr;
  decltype(&cuMemGetAddressRange) memGetAddressRange = nullptr;
};

// Returns the process-wide table; `ok` is false when no driver is present.
const DriverApi& driverApi();
const char* driverErrorString(CUresult r);

}  // namespace uccl
