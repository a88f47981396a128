/*
 * uccl_net.h -- network transport plugin interface.
 *
 * A plugin is a shared object that exports one symbol, `ucclNetPlugin_v1`, of type ucclNet_t.
 * The table has the same seventeen slots, in the same order, as the upstream project's
 * (src/include/uccl_net.h:22-64), so a plugin built against either header loads in both.
 * The proxy thread is the only caller of isend/irecv/test/progress.
 */
#ifndef UCCL_NET_PUBLIC_H_
#define UCCL_NET_PUBLIC_H_

#include "uccl.h"

#ifdef __cplusplus
extern "C" {
#endif

#define UCCL_NET_HANDLE_BYTES 128 /* size of the opaque address blob listen() fills */

typedef struct {
  char name[256];
  int pciPath;
  int guid;
  int ptrSupport; /* UCCL_PTR_HOST | UCCL_PTR_DEVICE */
  int speed;      /* MB/s */
  int latency;    /* ns */
  int maxComms;
} ucclNetProperties_t;

typedef struct {
  const char* name;

  ucclResult_t (*init)(void** handle);
  ucclResult_t (*finalize)(void* handle);

  ucclResult_t (*devices)(int* ndev);
  ucclResult_t (*getProperties)(int dev, ucclNetProperties_t* props);

  /* listen() writes an address blob of at most UCCL_NET_HANDLE_BYTES into listenAddr;
   * the peer hands that blob to connect().  accept() may return ucclInProgress. */
  ucclResult_t (*listen)(void* handle, void* listenAddr, void** listenComm);
  ucclResult_t (*connect)(void* handle, void* connectAddr, void** sendComm);
  ucclResult_t (*accept)(void* listenComm, void** recvComm);

  ucclResult_t (*regMr)(void* comm, void* data, size_t size, int type, void** mhandle);
  ucclResult_t (*deregMr)(void* comm, void* mhandle);

  /* Both may complete immediately; they still return a non-NULL request that test()
   * reports as done, so a caller can tell "posted" from "not posted". */
  ucclResult_t (*isend)(void* sendComm, void* data, size_t size, void* mhandle, void** request);
  ucclResult_t (*irecv)(void* recvComm, void* data, size_t size, void* mhandle, void** request);
  ucclResult_t (*test)(void* request, int* done, int* size);

  ucclResult_t (*closeSend)(void* sendComm);
  ucclResult_t (*closeRecv)(void* recvComm);
  ucclResult_t (*closeListen)(void* listenComm);

  ucclResult_t (*progress)(void* handle);
  ucclResult_t (*setTag)(void* comm, uint64_t tag);
} ucclNet_t;

#define UCCL_NET_PLUGIN_SYMBOL "ucclNetPlugin_v1"

#ifdef __cplusplus
}
#endif
#endif /* UCCL_NET_PUBLIC_H_ */
