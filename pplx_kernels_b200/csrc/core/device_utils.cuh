// Small device-side building blocks: warp reductions, a block-wide exclusive
// scan over a shared-memory array, and an upper-bound search in a prefix array.
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

// In-place exclusive scan of data[0..n) in shared memory; data[n] receives the
// total.  All threads of the block must call it; `warp_tmp` is 33 words of shared
// memory.  Ends with a __syncthreads().  blockDim.x must be a multiple of 32 and
// at most 1024.
__device__ inline void block_exclusive_scan(uint32_t* data, int n, uint32_t* warp_tmp) {
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  if (tid == 0) warp_tmp[32] = 0;  // running carry
  __syncthreads();
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + tid;
    const uint32_t v = (i < n) ? data[i] : 0u;
    const uint32_t inc = warp_inclusive_scan(v, lane);
    if (lane == 31) warp_tmp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      const uint32_t w = (lane < nwarps) ? warp_tmp[lane] : 0u;
      const uint32_t winc = warp_inclusive_scan(w, lane);
      warp_tmp[lane] = winc - w;  // exclusive offset of each warp
      if (lane == 31) warp_tmp[33] = winc;  // chunk total
    }
    __syncthreads();
    const uint32_t carry = warp_tmp[32];
    if (i < n) data[i] = carry + warp_tmp[warp] + inc - v;
    __syncthreads();
    if (tid == 0) warp_tmp[32] = carry + warp_tmp[33];
    __syncthreads();
  }
  if (tid == 0) data[n] = warp_tmp[32];
  __syncthreads();
}
constexpr int kScanTmpWords = 34;

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
