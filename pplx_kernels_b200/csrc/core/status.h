// Error record shared by host and device.
//
// The reference has no failure reporting: every device wait is an unbounded
// spin (intranode_dispatch.cu:87-88, 214-215; intranode_combine.cu:135-136) and
// device asserts are compiled out (device_utils.cuh:5).  Here each wait has a
// wall-clock limit; when it runs out, or when a bounds check fails, the kernel
// records the first failure in a `Status` block and then returns normally.  The
// block exists twice: a copy in device memory, on which the kernels run their
// atomics and which tells later waits to give up quickly, and a mirror in mapped
// pinned host memory that the thread which recorded the first failure fills in
// (fields first, then a system-scope fence, then `code`).  The host reads the
// mirror without synchronising with the device, so a failure is visible while
// other kernels are still inside their waits, and `dispatch()` / `combine()`
// refuse to launch on an object whose mirror is non-zero.
#pragma once

#include <cstdint>

namespace pplx {

enum StatusCode : uint32_t {
  kOk = 0,
  kTimeout = 1,       // a wait ran out; `phase`/`peer`/`expected`/`observed` say which
  kBadExpert = 2,     // an expert index >= num_experts
  kSlotOverflow = 3,  // a sender reserved a staging slot beyond its region
  kRowOverflow = 4,   // a receiver reserved an output row beyond the capacity
  kBadToken = 5,      // a trailer named a token index >= max_num_tokens
  kOutOfOrder = 6,    // two dispatches (or two combines) in a row on one object
};

enum Phase : uint32_t {
  kPhaseNone = 0,
  kPhaseDispatchCounts = 1,   // waiting for a peer's per-expert counts
  kPhaseDispatchPayload = 2,  // waiting for a peer's token payload
  kPhaseCombinePayload = 3,   // waiting for expert outputs of one token
  kPhaseBarrier = 4,
  kPhaseTest = 5,             // the wait-helper self test
  kPhaseFusedGemm = 6,
};

struct Status {
  uint32_t code;      // StatusCode of the first failure, 0 if none
  uint32_t phase;     // Phase
  uint32_t peer;      // source rank / token the wait was about
  uint32_t expected;
  uint32_t observed;
  uint32_t block;     // blockIdx.x of the reporter
  uint32_t rank;      // rank of the reporter
  uint32_t count;     // number of failures seen (first one wins the other fields)
  // Device copy only: device-side address of the host-visible mirror (0 = none).
  unsigned long long mirror;
};

}  // namespace pplx
