// Version and error-string entry points (reference: src/init.cc:37-45 and :272-288).
#include "uccl.h"

extern "C" ucclResult_t ucclGetVersion(int* version) {
  if (!version) return ucclInvalidArgument;
  *version = UCCL_VERSION;
  return ucclSuccess;
}

extern "C" const char* ucclGetErrorString(ucclResult_t result) {
  switch (result) {
    case ucclSuccess: return "no error";
    case ucclSystemError: return "unhandled system error (CUDA, socket or OS call failed)";
    case ucclInternalError: return "internal error";
    case ucclInvalidArgument: return "invalid argument";
    case ucclInvalidUsage: return "invalid usage";
    case ucclRemoteError: return "remote process exited, timed out or reported an error";
    case ucclInProgress: return "operation in progress";
    default: return "unknown result code";
  }
}
