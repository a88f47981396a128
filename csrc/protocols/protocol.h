// Wire protocols of the ring algorithms.
//
//  Simple : bulk data in step buffers, one flag per step (head/tail counters), highest bandwidth.
//  LL128  : 128-byte lines of sixteen 64-bit words; words 7 and 15 carry a sequence flag and the
//           other fourteen carry payload (112 of 128 bytes = 87.5 % efficiency).  A line is valid
//           when both flags equal the expected sequence number, so data and synchronisation travel
//           in the same store and no separate flag write or fence is needed.
//
// The constants match the reference's (src/protocols/protocol.h:15-33: Simple 4 MiB buffer,
// 2 slices x 4 steps; LL128 16 elements per line, 14 data + 2 flags, 1 MiB buffer).  The host
// codec below is the counterpart of src/protocols/ll128.cc:38-225 and is the executable
// specification the GPU ring kernel's LL128 path is tested against.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "uccl.h"

namespace uccl {

struct ProtoSimple {
  static constexpr int SlicePerChunk = 2;
  static constexpr int StepPerSlice = 4;
  static constexpr size_t DefaultBuffSize = 4u << 20;
};

struct ProtoLL128 {
  static constexpr int LineElems = 16;  // 64-bit words per line
  static constexpr int DataElems = 14;
  static constexpr int FlagElems = 2;
  static constexpr int LineSize = 128;  // bytes
  static constexpr int DataBytes = DataElems * 8;
  static constexpr size_t DefaultBuffSize = 1u << 20;
  static constexpr int FlagIdx0 = 7;
  static constexpr int FlagIdx1 = 15;
};

// Lines needed to carry `bytes` of payload.
inline size_t ll128LinesFor(size_t bytes) { return (bytes + ProtoLL128::DataBytes - 1) / ProtoLL128::DataBytes; }

// Writes one line: up to 112 payload bytes (zero padded), then both flags with release order.
void ll128PackLine(uint64_t* line, const void* data, size_t bytes, uint64_t seq);
// Spins (at most maxSpins polls) until both flags equal `seq`, then copies `bytes` of payload.
// Returns false if the line never became valid.
bool ll128UnpackLine(const uint64_t* line, void* data, size_t bytes, uint64_t seq, uint64_t maxSpins);

// Whole-buffer helpers: the buffer must hold ll128LinesFor(bytes) lines.
ucclResult_t ll128ProtocolSend(uint64_t* buffer, size_t bufferBytes, const void* data, size_t bytes, uint64_t seq);
ucclResult_t ll128ProtocolRecv(const uint64_t* buffer, size_t bufferBytes, void* data, size_t bytes, uint64_t seq,
                               uint64_t maxSpinsPerLine = 10000000ull);

}  // namespace uccl
