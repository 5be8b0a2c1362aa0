// Bounded device-side waits and failure reporting.
//
// Every spin on a word that another rank (or another block) writes goes through
// `wait_until`.  It polls with ld.acquire.sys; after a short burst of fast
// polls it starts reading %globaltimer every few polls and gives up once the
// limit has passed, recording what it waited for in the `Status` block.  It
// also gives up early when another thread has already recorded a failure, so a
// kernel with many pending waits drains quickly instead of timing out once per
// wait.  The caller decides what to do when it returns false (all callers skip
// the work that depended on the wait and fall through to the end of the
// kernel); nothing traps and nothing hangs.
#pragma once

#include "ptx.cuh"
#include "status.h"

// Attribute of the cold paths (failure reporting, the patient part of a wait).  Inlined by
// default: building them out of line (-DPPLX_COLD_PATH=__noinline__) was measured to change
// nothing at 1 and 8 tokens and to cost 1.2 µs in the 128-token combine, whose polling loop
// then keeps its state in local memory.
#ifndef PPLX_COLD_PATH
#define PPLX_COLD_PATH __forceinline__
#endif

namespace pplx {

struct WaitCtx {
  Status* status;       // device memory
  uint64_t timeout_ns;  // limit for a single wait
  uint32_t rank;
};

static __device__ PPLX_COLD_PATH void report_failure(Status* st, uint32_t code, uint32_t phase,
                                                   uint32_t peer, uint32_t expected,
                                                   uint32_t observed, uint32_t rank) {
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->phase = phase;
    st->peer = peer;
    st->expected = expected;
    st->observed = observed;
    st->block = blockIdx.x;
    st->rank = rank;
    // Host-visible mirror: plain stores of the fields, then the code behind a fence, so
    // that a host that reads a non-zero code also reads the fields that belong to it.
    Status* host = reinterpret_cast<Status*>(st->mirror);
    if (host != nullptr) {
      host->phase = phase;
      host->peer = peer;
      host->expected = expected;
      host->observed = observed;
      host->block = blockIdx.x;
      host->rank = rank;
      host->count = 1u;
      __threadfence_system();
      *reinterpret_cast<volatile uint32_t*>(&host->code) = code;
    }
  }
  atomicAdd(&st->count, 1u);
}

__device__ __forceinline__ bool failed_already(const Status* st) {
  return ptx::ld_volatile(&st->code) != 0u;
}

struct PredNonZero {
  __device__ __forceinline__ bool operator()(uint32_t v) const { return v != 0u; }
};
struct PredEq {
  uint32_t want;
  __device__ __forceinline__ bool operator()(uint32_t v) const { return v == want; }
};
// v has reached `want` on a counter that only grows, compared modulo 2^32.
struct PredReached {
  uint32_t want;
  __device__ __forceinline__ bool operator()(uint32_t v) const {
    return static_cast<int32_t>(v - want) >= 0;
  }
};
struct PredGe {
  uint32_t want;
  __device__ __forceinline__ bool operator()(uint32_t v) const { return v >= want; }
};

// The patient part of a wait: polls in bursts, looks at the clock and at the failure record in
// between.  Kept out of line (see report_failure).
template <typename Pred>
__device__ PPLX_COLD_PATH bool wait_slow(const uint32_t* p, Pred pred, uint32_t& observed,
                                       const WaitCtx& w, uint32_t phase, uint32_t peer,
                                       uint32_t expected) {
  uint32_t v = 0;
  const uint64_t t0 = ptx::globaltimer_ns();
#pragma unroll 1
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      v = ptx::ld_acquire_sys(p);
      if (pred(v)) {
        observed = v;
        return true;
      }
    }
    if (failed_already(w.status)) break;
    if (ptx::globaltimer_ns() - t0 > w.timeout_ns) {
      report_failure(w.status, kTimeout, phase, peer, expected, v, w.rank);
      break;
    }
  }
  observed = v;
  return false;
}

template <typename Pred>
__device__ __forceinline__ bool wait_until(const uint32_t* p, Pred pred, uint32_t& observed,
                                           const WaitCtx& w, uint32_t phase, uint32_t peer,
                                           uint32_t expected) {
#pragma unroll 1
  for (int i = 0; i < 128; ++i) {
    const uint32_t v = ptx::ld_acquire_sys(p);
    if (pred(v)) {
      observed = v;
      return true;
    }
  }
  return wait_slow(p, pred, observed, w, phase, peer, expected);
}

}  // namespace pplx
