// Small stream-ordered collectives and utilities on symmetric memory.
//
// Role parity: nvshmemx_barrier_all_on_stream and nvshmemx_alltoallmem_on_stream
// as the reference uses them (bindings/nvshmem.cpp:64-80), and the sleep kernel
// of csrc/core/kernels.cu:8-20.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

#include "../core/status.h"
#include "a2a_params.h"

namespace pplx {

struct BarrierParams {
  uint8_t* peer[kMaxWorld];  // base of every rank's flag array: u32 [world], then counters
  uint8_t* mc;               // multicast alias of the flag arrays, or nullptr
  uint32_t* epoch;           // local device word, last completed epoch
  Status* status;
  uint64_t timeout_ns;
  int rank;
  int world;
};

// flags[rank] on every peer <- epoch + 1 (release), then wait until every local
// flag reached it.  With a multicast alias: one `multimem.red` adds 1 to word
// kBarrierMcWord of every rank, and the wait is for world * (epoch + 1) there.
constexpr int kBarrierMcWord = 32;
constexpr size_t kBarrierFlagBytes = 256;
cudaError_t launch_barrier(const BarrierParams& b, cudaStream_t stream);

struct AllToAllCopyParams {
  uint8_t* peer_dst[kMaxWorld];  // base of `dest` on every rank
  const uint8_t* src;            // local source, world chunks
  size_t chunk_bytes;            // multiple of 16
  int rank;
  int world;
};

// Chunk j of `src` -> chunk `rank` of rank j's `dest`.  Follow with a barrier.
cudaError_t launch_alltoall_copy(const AllToAllCopyParams& a, int blocks_per_peer,
                                 cudaStream_t stream);

// Occupies one thread for roughly `ns` nanoseconds.
cudaError_t launch_sleep(uint64_t ns, cudaStream_t stream);

// Waits (bounded by `timeout_ns`) for *flag != 0 and records the outcome in
// `status`.  Lets a test see the time-out path return cleanly.
cudaError_t launch_wait_probe(const uint32_t* flag, Status* status, uint64_t timeout_ns,
                              cudaStream_t stream);

}  // namespace pplx
