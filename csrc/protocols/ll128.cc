#include <string.h>

#include "protocol.h"

namespace uccl {

void ll128PackLine(uint64_t* line, const void* data, size_t bytes, uint64_t seq) {
  uint64_t words[ProtoLL128::DataElems] = {0};
  if (bytes > static_cast<size_t>(ProtoLL128::DataBytes)) bytes = ProtoLL128::DataBytes;
  if (bytes) memcpy(words, data, bytes);
  int w = 0;
  for (int i = 0; i < ProtoLL128::LineElems; ++i) {
    if (i == ProtoLL128::FlagIdx0 || i == ProtoLL128::FlagIdx1) continue;
    __atomic_store_n(&line[i], words[w++], __ATOMIC_RELAXED);
  }
  // payload before flags: a reader that sees both flags sees the fourteen data words
  __atomic_thread_fence(__ATOMIC_RELEASE);
  __atomic_store_n(&line[ProtoLL128::FlagIdx0], seq, __ATOMIC_RELEASE);
  __atomic_store_n(&line[ProtoLL128::FlagIdx1], seq, __ATOMIC_RELEASE);
}

bool ll128UnpackLine(const uint64_t* line, void* data, size_t bytes, uint64_t seq, uint64_t maxSpins) {
  uint64_t spins = 0;
  while (true) {
    const uint64_t f0 = __atomic_load_n(&line[ProtoLL128::FlagIdx0], __ATOMIC_ACQUIRE);
    const uint64_t f1 = __atomic_load_n(&line[ProtoLL128::FlagIdx1], __ATOMIC_ACQUIRE);
    if (f0 == seq && f1 == seq) break;
    if (++spins > maxSpins) return false;
  }
  uint64_t words[ProtoLL128::DataElems];
  int w = 0;
  for (int i = 0; i < ProtoLL128::LineElems; ++i) {
    if (i == ProtoLL128::FlagIdx0 || i == ProtoLL128::FlagIdx1) continue;
    words[w++] = __atomic_load_n(&line[i], __ATOMIC_RELAXED);
  }
  if (bytes > static_cast<size_t>(ProtoLL128::DataBytes)) bytes = ProtoLL128::DataBytes;
  if (bytes) memcpy(data, words, bytes);
  return true;
}

ucclResult_t ll128ProtocolSend(uint64_t* buffer, size_t bufferBytes, const void* data, size_t bytes, uint64_t seq) {
  if (!buffer || (bytes && !data) || seq == 0) return ucclInvalidArgument;
  const size_t lines = ll128LinesFor(bytes);
  if (lines * ProtoLL128::LineSize > bufferBytes) return ucclInvalidArgument;
  const char* p = static_cast<const char*>(data);
  for (size_t l = 0; l < lines; ++l) {
    const size_t off = l * ProtoLL128::DataBytes;
    const size_t n = bytes - off < static_cast<size_t>(ProtoLL128::DataBytes) ? bytes - off : ProtoLL128::DataBytes;
    ll128PackLine(buffer + l * ProtoLL128::LineElems, p + off, n, seq);
  }
  return ucclSuccess;
}

ucclResult_t ll128ProtocolRecv(const uint64_t* buffer, size_t bufferBytes, void* data, size_t bytes, uint64_t seq,
                               uint64_t maxSpinsPerLine) {
  if (!buffer || (bytes && !data) || seq == 0) return ucclInvalidArgument;
  const size_t lines = ll128LinesFor(bytes);
  if (lines * ProtoLL128::LineSize > bufferBytes) return ucclInvalidArgument;
  char* p = static_cast<char*>(data);
  for (size_t l = 0; l < lines; ++l) {
    const size_t off = l * ProtoLL128::DataBytes;
    const size_t n = bytes - off < static_cast<size_t>(ProtoLL128::DataBytes) ? bytes - off : ProtoLL128::DataBytes;
    if (!ll128UnpackLine(buffer + l * ProtoLL128::LineElems, p + off, n, seq, maxSpinsPerLine)) return ucclRemoteError;
  }
  return ucclSuccess;
}

}  // namespace uccl
