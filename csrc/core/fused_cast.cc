// Collectives with a fused sum / scale / cast epilogue: ucclReduceScatterEx and ucclAllReduceEx.
// out = cast<outType>(scale * sum over ranks(in)), the sum carried in fp32 from the peer loads to
// the store (csrc/kernels/fused_cast.cu).  The reference has neither a scale nor a second element
// type on any collective; it adds in the 16-bit type (src/device/reduce_kernel.hpp:17-20) and
// lists further types as future work (desgin/design-spec.md:1759).
#include <string.h>

#include <algorithm>

#include "../kernels/collectives.cuh"
#include "enqueue.h"
#include "log.h"

using namespace uccl;

namespace {

struct DeviceGuard {
  int prev = -1, want;
  explicit DeviceGuard(int dev) : want(dev) {
    cudaGetDevice(&prev);
    if (prev != want) cudaSetDevice(want);
  }
  ~DeviceGuard() {
    if (prev >= 0 && prev != want) cudaSetDevice(prev);
  }
};

bool reducibleIn(ucclDataType_t t) { return t == ucclFloat16 || t == ucclBfloat16 || t == ucclFloat32; }
bool castOut(ucclDataType_t t) { return reducibleIn(t) || t == ucclFloat8e4m3; }

ucclResult_t validateEx(Comm* c, ucclDataType_t inType, ucclDataType_t outType, const void* send, void* recv,
                        const float* blockScales) {
  if (!commValid(c)) return ucclInvalidArgument;
  if (c->abortFlag.load()) return ucclInvalidUsage;
  const int ae = c->asyncError.load();
  if (ae != ucclSuccess) return static_cast<ucclResult_t>(ae);
  if (!reducibleIn(inType) || !castOut(outType)) return ucclInvalidArgument;
  if (!send || !recv || (outType == ucclFloat8e4m3 && !blockScales)) return ucclInvalidArgument;
  if (groupActive()) {
    commSetError(c, "the fused-epilogue collectives cannot be deferred into a group");
    return ucclInvalidUsage;
  }
  if (c->backend != BACKEND_CUDA || (c->nRanks > 1 && (!c->p2pReady || c->useNet))) {
    commSetError(c, "the fused-epilogue collectives need GPU ranks in one NVLink domain");
    return ucclInvalidUsage;
  }
  return ucclSuccess;
}

// elements per 16-byte vector of the input type; chunks are whole vectors (and whole 128-element
// scale blocks for fp8 output)
size_t granule(ucclDataType_t inType, ucclDataType_t outType) {
  if (outType == ucclFloat8e4m3) return 128;
  return 16 / dataTypeSize(inType);
}

}  // namespace

extern "C" ucclResult_t ucclReduceScatterEx(const void* sendbuff, void* recvbuff, size_t recvcount,
                                            ucclDataType_t inType, ucclDataType_t outType, float scale,
                                            float* blockScales, ucclComm_t comm, void* stream) {
  Comm* c = toComm(comm);
  ucclResult_t r = validateEx(c, inType, outType, sendbuff, recvbuff, blockScales);
  if (r != ucclSuccess) return r;
  if (recvcount == 0) return ucclSuccess;
  const size_t g = granule(inType, outType);
  if (recvcount % g != 0 || (reinterpret_cast<uintptr_t>(recvbuff) & 15) || (reinterpret_cast<uintptr_t>(sendbuff) & 15)) {
    commSetError(c, "fused-epilogue reduce-scatter needs 16-byte aligned buffers and recvcount a multiple of %zu", g);
    return ucclInvalidArgument;
  }
  DeviceGuard guard(c->cudaDev);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int n = c->nRanks == 1 ? 1 : c->localRanks;
  const size_t es = dataTypeSize(inType);
  const size_t chunkBytes = recvcount * es;
  const size_t outEs = dataTypeSize(outType);
  commCount(c, ucclCollReduceScatter, chunkBytes * n, ucclAlgoTwoShot);
  int blocks = c->cfg.maxCtas > 0 ? std::min(c->cfg.maxCtas, kMaxBlocks) : kMaxBlocks;
  if (c->forcedBlocks > 0) blocks = std::min(c->forcedBlocks, kMaxBlocks);
  blocks = static_cast<int>(std::max<size_t>(1, std::min<size_t>(blocks, (recvcount + 4095) / 4096)));

  CastArgs a;
  memset(&a, 0, sizeof(a));
  a.dc = c->dev;
  a.inType = inType;
  a.outType = outType;
  a.scale = scale;
  if (n == 1) {
    a.dc.rank = 0;
    a.dc.nranks = 1;
    a.in[0] = static_cast<const char*>(sendbuff);
    a.chunkStride = chunkBytes;
    a.chunkElems = recvcount;
    a.out = static_cast<char*>(recvbuff);
    a.outScales = blockScales;
    if (launchReduceCastKernel(a, blocks, s) != cudaSuccess) return ucclSystemError;
    return ucclSuccess;
  }
  SymSegment* seg = c->heap.find(sendbuff, chunkBytes * n);
  if (seg) {
    const size_t off = static_cast<size_t>(static_cast<const char*>(sendbuff) - seg->local);
    for (int p = 0; p < n; ++p) a.in[p] = seg->peer[p] + off;
    // through the switch only when asked for: its result comes back rounded to the input type
    if (c->forcedAlgo == ucclAlgoNvls && seg->mc) a.inMc = seg->mc + off;
    a.chunkStride = chunkBytes;
    a.chunkElems = recvcount;
    a.out = static_cast<char*>(recvbuff);
    a.outScales = blockScales;
    if (launchReduceCastKernel(a, blocks, s) != cudaSuccess) {
      commSetError(c, "kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
      return ucclSystemError;
    }
    return ucclSuccess;
  }
  // staged: pieces of every rank chunk travel through the arena's staging area
  const size_t stageOff = stagingOffset(c);
  const size_t stageBytes = c->cfg.stagingBytes & ~size_t(4095);
  const size_t capElems = ((stageBytes / n) / (128 * es)) * 128;  // whole scale blocks per piece
  if (capElems == 0) {
    commSetError(c, "staging area too small; raise UCCL_STAGING_BYTES or pass a buffer from ucclMemAlloc");
    return ucclInvalidUsage;
  }
  for (size_t eo = 0; eo < recvcount; eo += capElems) {
    const size_t len = std::min(capElems, recvcount - eo);
    for (int p = 0; p < n; ++p) a.in[p] = c->arena->peer[p] + stageOff;
    a.inMc = nullptr;
    a.inUser = static_cast<const char*>(sendbuff) + eo * es;
    a.inStride = chunkBytes;
    a.chunkStride = capElems * es;
    a.chunkElems = len;
    a.out = static_cast<char*>(recvbuff) + eo * outEs;
    a.outScales = blockScales ? blockScales + eo / 128 : nullptr;
    if (launchReduceCastKernel(a, blocks, s) != cudaSuccess) {
      commSetError(c, "kernel launch failed: %s", cudaGetErrorString(cudaGetLastError()));
      return ucclSystemError;
    }
  }
  return ucclSuccess;
}

extern "C" ucclResult_t ucclAllReduceEx(const void* sendbuff, void* recvbuff, size_t count, ucclDataType_t inType,
                                        ucclDataType_t outType, float scale, float* blockScales, ucclComm_t comm,
                                        void* stream) {
  Comm* c = toComm(comm);
  ucclResult_t r = validateEx(c, inType, outType, sendbuff, recvbuff, blockScales);
  if (r != ucclSuccess) return r;
  if (count == 0) return ucclSuccess;
  const int n = c->nRanks == 1 ? 1 : c->localRanks;
  const size_t g = granule(inType, outType);
  if (count % (g * n) != 0) {
    commSetError(c, "fused-epilogue all-reduce needs count to be a multiple of %zu (granule x ranks)", g * n);
    return ucclInvalidArgument;
  }
  if ((reinterpret_cast<uintptr_t>(recvbuff) & 15) || (blockScales && (reinterpret_cast<uintptr_t>(blockScales) & 15)))
    return ucclInvalidArgument;
  // reduce + scale + cast my shard straight into its place in the output, then gather the shards
  // (and the scales) in the output type: the second half moves the narrow elements
  const size_t per = count / n;
  const size_t outEs = dataTypeSize(outType);
  char* out = static_cast<char*>(recvbuff);
  const int me = n == 1 ? 0 : c->localRank;
  float* myScales = blockScales ? blockScales + static_cast<size_t>(me) * (per / 128) : nullptr;
  r = ucclReduceScatterEx(sendbuff, out + static_cast<size_t>(me) * per * outEs, per, inType, outType, scale, myScales, comm, stream);
  if (r != ucclSuccess || n == 1) return r;
  r = ucclAllGather(out + static_cast<size_t>(me) * per * outEs, out, per * outEs, ucclUint8, comm, stream);
  if (r != ucclSuccess) return r;
  if (blockScales) r = ucclAllGather(myScales, blockScales, per / 128, ucclFloat32, comm, stream);
  return r;
}
