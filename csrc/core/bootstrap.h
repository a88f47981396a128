// Out-of-band control plane: TCP rendezvous + ring all-gather + tagged point-to-point
// messages + file-descriptor passing between ranks of one host.
//
// The reference bootstraps over MPI (src/bootstrap.cc:24-127: MPI_Init_thread, rank/size from
// MPI_COMM_WORLD, MPI_Allgather, MPI_Barrier) and its 128-byte unique id carries no address
// (src/init.cc:47-61).  There is no MPI on the target machines, so here the unique id holds the
// socket address of a rendezvous service started by ucclGetUniqueId, the way NCCL does it:
//   1. every rank opens a listening socket and reports {rank, address} to the root service,
//   2. the service answers each rank with the whole address table and retires,
//   3. ranks connect in a ring (rank -> rank+1) for all-gather / barrier, and open short-lived
//      connections for tagged messages,
//   4. ranks on one host own an abstract AF_UNIX datagram socket for SCM_RIGHTS fd passing
//      (used to share CUDA VMM allocation handles).
// Every blocking step has a deadline and watches the communicator's abort word.
#pragma once
#include <netinet/in.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "config.h"
#include "uccl.h"

namespace uccl {

struct BootstrapIdPayload {
  uint64_t magic;
  uint32_t version;
  uint32_t pid;
  uint8_t nonce[16];
  struct sockaddr_in addr;
  uint8_t pad[UCCL_UNIQUE_ID_BYTES - 8 - 4 - 4 - 16 - sizeof(struct sockaddr_in)];
};
static_assert(sizeof(BootstrapIdPayload) == UCCL_UNIQUE_ID_BYTES, "id payload must fill the unique id");

constexpr uint64_t kBootstrapMagic = 0x5543434c42323030ull;  // "UCCLB200"

// Starts the rendezvous service thread and fills `id` with its address.
ucclResult_t bootstrapCreateRoot(ucclUniqueId* id, const Config& cfg);
// Builds an id that points at a service somebody else runs at ip:port with the given nonce
// seed (used when all ranks derive the id from a shared host:port string).
ucclResult_t bootstrapIdFromAddress(const char* ip, int port, uint64_t seed, ucclUniqueId* id);
// Runs the rendezvous service for `id` on the caller's thread-less background (detached).
ucclResult_t bootstrapServeId(const ucclUniqueId& id, const Config& cfg);

class Bootstrap {
 public:
  Bootstrap() = default;
  ~Bootstrap();
  Bootstrap(const Bootstrap&) = delete;
  Bootstrap& operator=(const Bootstrap&) = delete;

  ucclResult_t init(const ucclUniqueId& id, int rank, int nranks, const Config& cfg,
                    const std::atomic<uint32_t>* abortFlag);
  // data holds nranks * bytes; slot [rank] is the input, all slots are filled on return.
  ucclResult_t allGather(void* data, size_t bytes);
  ucclResult_t barrier();
  ucclResult_t send(int peer, int tag, const void* data, size_t bytes);
  ucclResult_t recv(int peer, int tag, void* data, size_t bytes);
  // Same-host only.
  ucclResult_t sendFd(int peer, int tag, int fd);
  ucclResult_t recvFd(int peer, int tag, int* fd);
  void close();

  int rank() const { return rank_; }
  int nranks() const { return nranks_; }
  const std::string& lastError() const { return err_; }

 private:
  ucclResult_t fail(ucclResult_t r, const char* fmt, ...) __attribute__((format(printf, 3, 4)));
  bool expired(uint64_t deadlineMs) const;
  uint64_t deadline() const;
  int acceptOne(uint64_t deadlineMs, int* srcRank, int* tag, uint64_t* size);
  ucclResult_t ioAll(int fd, void* buf, size_t len, bool isSend, uint64_t deadlineMs);
  ucclResult_t duplex(int sfd, const void* sbuf, int rfd, void* rbuf, size_t len, uint64_t deadlineMs);

  int rank_ = -1, nranks_ = 0;
  uint64_t timeoutMs_ = 60000;
  const std::atomic<uint32_t>* abort_ = nullptr;
  uint8_t nonce_[16] = {};
  int listenFd_ = -1;
  int nextFd_ = -1, prevFd_ = -1;
  int unixFd_ = -1;
  std::vector<struct sockaddr_in> peers_;
  // stashed unexpected messages / fds keyed by (src, tag)
  std::map<std::pair<int, int>, std::vector<std::vector<uint8_t>>> stash_;
  std::map<std::pair<int, int>, std::vector<int>> fdStash_;
  std::string err_;
};

// Helpers shared with the socket network plugin.
int pickInterfaceAddr(const std::string& ifname, struct in_addr* out);
uint64_t nowMs();

}  // namespace uccl
