// Geometry of flag-in-data transfer lines, for host and device code (see ll128.cuh).
#pragma once

namespace pplx {
namespace ll {

constexpr int kLineBytes = 128;  // one line on the wire
constexpr int kLineData = 120;   // payload bytes in it; the last 8 bytes are the flag

// Lines needed for `bytes` of payload.
constexpr int lines_for(int bytes) { return (bytes + kLineData - 1) / kLineData; }

}  // namespace ll
}  // namespace pplx
