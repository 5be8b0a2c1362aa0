#include "collectives.h"

#include "../core/ptx.cuh"
#include "../core/wait.cuh"

namespace pplx {
namespace {

__global__ void barrier_kernel(const __grid_constant__ BarrierParams b) {
  const int tid = threadIdx.x;
  const uint32_t target = ptx::ld_volatile(b.epoch) + 1u;
  __syncthreads();
  // Epochs only grow; compare modulo 2^32.
  struct Reached {
    uint32_t t;
    __device__ bool operator()(uint32_t v) const { return static_cast<int32_t>(v - t) >= 0; }
  };
  if (b.mc != nullptr) {
    if (tid == 0) {
      ptx::multimem_red_add_release_sys(reinterpret_cast<uint32_t*>(b.mc) + kBarrierMcWord, 1u);
      const uint32_t* mine = reinterpret_cast<const uint32_t*>(b.peer[b.rank]) + kBarrierMcWord;
      const WaitCtx w{b.status, b.timeout_ns, static_cast<uint32_t>(b.rank)};
      const uint32_t want = target * static_cast<uint32_t>(b.world);
      uint32_t seen;
      wait_until(mine, Reached{want}, seen, w, kPhaseBarrier, 0u, want);
    }
  } else if (tid < b.world) {
    uint32_t* remote = reinterpret_cast<uint32_t*>(b.peer[tid]) + b.rank;
    ptx::st_release_sys(remote, target);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(b.peer[b.rank]) + tid;
    const WaitCtx w{b.status, b.timeout_ns, static_cast<uint32_t>(b.rank)};
    uint32_t seen;
    wait_until(mine, Reached{target}, seen, w, kPhaseBarrier, tid, target);
  }
  __syncthreads();
  if (tid == 0) *b.epoch = target;
}

__global__ void alltoall_copy_kernel(const __grid_constant__ AllToAllCopyParams a) {
  const int dst_rank = blockIdx.y;
  const size_t nvec = a.chunk_bytes >> 4;
  const int4* src = reinterpret_cast<const int4*>(a.src + dst_rank * a.chunk_bytes);
  int4* dst = reinterpret_cast<int4*>(a.peer_dst[dst_rank] + a.rank * a.chunk_bytes);
  // Eight 16-byte loads in flight per thread before the first store, so that the copy is
  // bound by the link and not by one memory latency per vector.
  constexpr int kBatch = 8;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t v0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v0 < nvec;
       v0 += stride * kBatch) {
    int4 r[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const size_t v = v0 + u * stride;
      if (v < nvec) r[u] = ptx::ld_nc_v4(src + v);
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const size_t v = v0 + u * stride;
      if (v < nvec) ptx::st_v4(dst + v, r[u]);
    }
  }
}

__global__ void sleep_kernel(uint64_t ns) {
  const uint64_t t0 = ptx::globaltimer_ns();
  while (ptx::globaltimer_ns() - t0 < ns) ptx::nanosleep(1000);
}

__global__ void wait_probe_kernel(const uint32_t* flag, Status* status, uint64_t timeout_ns) {
  const WaitCtx w{status, timeout_ns, 0u};
  uint32_t seen;
  wait_until(flag, PredNonZero{}, seen, w, kPhaseTest, 0u, 1u);
}

}  // namespace

cudaError_t launch_barrier(const BarrierParams& b, cudaStream_t stream) {
  barrier_kernel<<<1, 32 * ((b.world + 31) / 32), 0, stream>>>(b);
  return cudaGetLastError();
}

cudaError_t launch_alltoall_copy(const AllToAllCopyParams& a, int blocks_per_peer,
                                 cudaStream_t stream) {
  if (a.chunk_bytes % 16 != 0) return cudaErrorInvalidValue;
  alltoall_copy_kernel<<<dim3(blocks_per_peer, a.world), 512, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_sleep(uint64_t ns, cudaStream_t stream) {
  sleep_kernel<<<1, 1, 0, stream>>>(ns);
  return cudaGetLastError();
}

cudaError_t launch_wait_probe(const uint32_t* flag, Status* status, uint64_t timeout_ns,
                              cudaStream_t stream) {
  wait_probe_kernel<<<1, 1, 0, stream>>>(flag, status, timeout_ns);
  return cudaGetLastError();
}

}  // namespace pplx
