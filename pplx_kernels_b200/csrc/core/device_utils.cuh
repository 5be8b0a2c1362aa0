// Small device-side building blocks: warp reductions, a one-warp exclusive scan
// over a shared-memory array, and an upper-bound search in a prefix array.
//
// Role parity: csrc/core/device_utils.cuh:19-57 of the reference (warp_sum,
// warp_and, half_warp_reduce_max).
#pragma once

#include <cstdint>

namespace pplx {

__device__ __forceinline__ uint32_t warp_sum(uint32_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ bool warp_and(bool v) {
  return __all_sync(0xffffffffu, v);
}

__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  return v;
}

// Exclusive scan of data[0..n) in shared memory by ONE warp (all 32 lanes call
// it); data[n] receives the total when `write_total`.  Each lane owns a
// contiguous run, so n up to a few thousand costs a handful of steps and no
// block barrier.  The caller synchronises the block afterwards.
__device__ __forceinline__ void warp_exclusive_scan_smem(uint32_t* data, int n, int lane,
                                                         bool write_total) {
  const int per = (n + 31) >> 5;
  const int begin = min(lane * per, n);
  const int end = min(begin + per, n);
  uint32_t sum = 0;
  for (int i = begin; i < end; ++i) sum += data[i];
  const uint32_t inc = warp_inclusive_scan(sum, lane);
  uint32_t run = inc - sum;
  for (int i = begin; i < end; ++i) {
    const uint32_t v = data[i];
    data[i] = run;
    run += v;
  }
  if (write_total && lane == 31) data[n] = inc;
  __syncwarp();
}

// Largest p in [0, n) with prefix[p] <= x, given prefix[0] = 0 and x < prefix[n].
// Entries with equal prefix (empty groups) are skipped in favour of the last one.
__device__ __forceinline__ int find_group(const uint32_t* prefix, int n, uint32_t x) {
  int lo = 0, hi = n;  // invariant: prefix[lo] <= x < prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= x) lo = mid;
    else hi = mid;
  }
  return lo;
}

}  // namespace pplx
