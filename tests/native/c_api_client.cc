// A plain C++ client of the public C ABI (include/uccl.h), no Python in between.
//
//   c_api_client rank <rank> <nranks> <idfile>   one process per rank; rank 0 creates the unique
//                                                id and publishes it through <idfile>
//   c_api_client initall <ndev>                  one process, ucclCommInitAll, one thread per rank
//
// Both modes run the reference's integration check (tests/cpp/test_allreduce.cc:37-144): fp16
// all-reduce at counts 1 ... 1 Mi where rank r contributes r + 1 and every element must come back
// as n (n + 1) / 2, then bf16 at 1024 elements; plus all-gather and reduce-scatter, which the
// reference's client never calls.  Buffers live on the GPU (device = rank % visible devices)
// unless UCCL_BACKEND=cpu or no device is visible, in which case they are host memory and the
// ranks are CPU ranks.  Exit code 0 = every check passed; each rank prints one line.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>
#include <unistd.h>

#include <atomic>
#include <cmath>
#include <string>
#include <thread>
#include <vector>

#include "uccl.h"

namespace {

bool g_onGpu = false;

#define CHECK_UCCL(call)                                                                              \
  do {                                                                                                \
    ucclResult_t r_ = (call);                                                                         \
    if (r_ != ucclSuccess) {                                                                          \
      fprintf(stderr, "%s:%d %s -> %s (%s)\n", __FILE__, __LINE__, #call, ucclGetErrorString(r_),     \
              ucclGetLastError(nullptr));                                                             \
      return 1;                                                                                       \
    }                                                                                                 \
  } while (0)

struct Buffer {
  void* p = nullptr;
  size_t bytes = 0;
  explicit Buffer(size_t b) : bytes(b) {
    if (b == 0) return;
    if (g_onGpu) {
      if (cudaMalloc(&p, b) != cudaSuccess) p = nullptr;
    } else {
      p = malloc(b);
    }
  }
  ~Buffer() {
    if (!p) return;
    if (g_onGpu) cudaFree(p);
    else free(p);
  }
  void upload(const void* src) {
    if (g_onGpu) cudaMemcpy(p, src, bytes, cudaMemcpyHostToDevice);
    else memcpy(p, src, bytes);
  }
  void download(void* dst) {
    if (g_onGpu) cudaMemcpy(dst, p, bytes, cudaMemcpyDeviceToHost);
    else memcpy(dst, p, bytes);
  }
};

int syncStream(cudaStream_t s) {
  if (!g_onGpu) return 0;
  return cudaStreamSynchronize(s) == cudaSuccess ? 0 : 1;
}

// the checks of one rank; `stream` is a CUDA stream on GPU ranks and NULL on CPU ranks
int runChecks(ucclComm_t comm, int rank, int n, cudaStream_t stream) {
  int count = 0, me = -1;
  CHECK_UCCL(ucclCommCount(comm, &count));
  CHECK_UCCL(ucclCommUserRank(comm, &me));
  if (count != n || me != rank) {
    fprintf(stderr, "rank %d: count/rank mismatch (%d, %d)\n", rank, count, me);
    return 1;
  }
  const float expect = n * (n + 1) / 2.0f;
  int errors = 0;
  const size_t counts[] = {1, 16, 256, 1024, 4096, 65536, 262144, 1048576};
  for (size_t cnt : counts) {
    std::vector<__half> h(cnt, __float2half(static_cast<float>(rank + 1)));
    Buffer b(cnt * sizeof(__half));
    if (!b.p) return 1;
    b.upload(h.data());
    CHECK_UCCL(ucclAllReduce(b.p, b.p, cnt, ucclFloat16, ucclSum, comm, stream));
    if (syncStream(stream)) return 1;
    b.download(h.data());
    for (size_t i = 0; i < cnt; ++i)
      if (std::fabs(__half2float(h[i]) - expect) > 0.1f) {
        if (errors < 5) fprintf(stderr, "rank %d: fp16 count %zu [%zu] = %f, want %f\n", rank, cnt, i, __half2float(h[i]), expect);
        ++errors;
        break;
      }
  }
  {
    const size_t cnt = 1024;
    std::vector<__nv_bfloat16> h(cnt, __float2bfloat16(static_cast<float>(rank + 1)));
    Buffer b(cnt * 2);
    b.upload(h.data());
    CHECK_UCCL(ucclAllReduce(b.p, b.p, cnt, ucclBfloat16, ucclSum, comm, stream));
    if (syncStream(stream)) return 1;
    b.download(h.data());
    for (size_t i = 0; i < cnt; ++i)
      if (std::fabs(__bfloat162float(h[i]) - expect) > 0.1f) {
        ++errors;
        break;
      }
  }
  {
    // all-gather and reduce-scatter, fp32, out of place, inside one group
    const size_t cnt = 3001;
    std::vector<float> mine(cnt, static_cast<float>(rank + 1)), all(cnt * n, 0.f), full(cnt * n), part(cnt, 0.f);
    for (size_t i = 0; i < cnt * n; ++i) full[i] = static_cast<float>((i % 7) + rank);
    Buffer bs(cnt * 4), br(cnt * n * 4), bf(cnt * n * 4), bp(cnt * 4);
    bs.upload(mine.data());
    bf.upload(full.data());
    CHECK_UCCL(ucclGroupStart());
    CHECK_UCCL(ucclAllGather(bs.p, br.p, cnt, ucclFloat32, comm, stream));
    CHECK_UCCL(ucclReduceScatter(bf.p, bp.p, cnt, ucclFloat32, ucclSum, comm, stream));
    CHECK_UCCL(ucclGroupEnd());
    if (syncStream(stream)) return 1;
    br.download(all.data());
    bp.download(part.data());
    for (size_t i = 0; i < cnt * n; ++i)
      if (all[i] != static_cast<float>(i / cnt + 1)) {
        ++errors;
        break;
      }
    for (size_t i = 0; i < cnt; ++i) {
      const size_t g = rank * cnt + i;
      const float want = n * static_cast<float>(g % 7) + n * (n - 1) / 2.0f;
      if (std::fabs(part[i] - want) > 1e-3f) {
        ++errors;
        break;
      }
    }
  }
  CHECK_UCCL(ucclCommFinalize(comm));
  printf("rank %d of %d (%s): %s\n", rank, n, g_onGpu ? "gpu" : "cpu", errors ? "FAILED" : "ok");
  fflush(stdout);
  return errors ? 1 : 0;
}

bool pickBackend(int* ndev) {
  const char* be = getenv("UCCL_BACKEND");
  *ndev = 0;
  if (be && (!strcasecmp(be, "cpu") || !strcasecmp(be, "host"))) return false;
  if (cudaGetDeviceCount(ndev) != cudaSuccess) {
    (void)cudaGetLastError();
    *ndev = 0;
  }
  return *ndev > 0;
}

int modeRank(int rank, int n, const char* idfile) {
  int ndev = 0;
  g_onGpu = pickBackend(&ndev);
  if (g_onGpu && cudaSetDevice(rank % ndev) != cudaSuccess) return 1;
  ucclUniqueId id;
  memset(&id, 0, sizeof(id));
  if (rank == 0) {
    CHECK_UCCL(ucclGetUniqueId(&id));
    const std::string tmp = std::string(idfile) + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f || fwrite(&id, sizeof(id), 1, f) != 1) return 1;
    fclose(f);
    if (rename(tmp.c_str(), idfile) != 0) return 1;
  } else {
    FILE* f = nullptr;
    for (int i = 0; i < 6000 && !(f = fopen(idfile, "rb")); ++i) usleep(10000);
    if (!f || fread(&id, sizeof(id), 1, f) != 1) {
      fprintf(stderr, "rank %d: unique id file never appeared\n", rank);
      return 1;
    }
    fclose(f);
  }
  ucclComm_t comm = nullptr;
  CHECK_UCCL(ucclCommInitRank(&comm, n, id, rank));
  cudaStream_t stream = nullptr;
  if (g_onGpu && cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) return 1;
  const int rc = runChecks(comm, rank, n, stream);
  CHECK_UCCL(ucclCommDestroy(comm));
  if (stream) cudaStreamDestroy(stream);
  return rc;
}

int modeInitAll(int n) {
  int ndev = 0;
  g_onGpu = pickBackend(&ndev);
  if (g_onGpu && ndev < n) {
    fprintf(stderr, "initall %d needs %d devices, %d visible\n", n, n, ndev);
    return 2;
  }
  std::vector<ucclComm_t> comms(n, nullptr);
  CHECK_UCCL(ucclCommInitAll(comms.data(), n, nullptr));
  std::atomic<int> failed{0};
  std::vector<std::thread> th;
  for (int r = 0; r < n; ++r)
    th.emplace_back([&, r] {
      cudaStream_t stream = nullptr;
      if (g_onGpu) {
        cudaSetDevice(r);
        cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
      }
      if (runChecks(comms[r], r, n, stream) != 0) failed.fetch_add(1);
      if (stream) cudaStreamDestroy(stream);
    });
  for (auto& t : th) t.join();
  // teardown is collective too: one thread per communicator
  std::vector<std::thread> td;
  for (int r = 0; r < n; ++r) td.emplace_back([&, r] { ucclCommDestroy(comms[r]); });
  for (auto& t : td) t.join();
  return failed.load() ? 1 : 0;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc == 5 && !strcmp(argv[1], "rank")) return modeRank(atoi(argv[2]), atoi(argv[3]), argv[4]);
  if (argc == 3 && !strcmp(argv[1], "initall")) return modeInitAll(atoi(argv[2]));
  fprintf(stderr, "usage: %s rank <rank> <nranks> <idfile> | initall <ndev>\n", argv[0]);
  return 64;
}
