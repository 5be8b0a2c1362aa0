// Inline-PTX primitives for system-scope signalling over NVLink peer memory.
//
// Role parity: the reference keeps five flag helpers in csrc/core/atomic.cuh:7-31
// (volatile ld/st, ld.acquire.sys, st.release.sys, atom.release.sys.add).  This
// header provides the same capabilities plus what the sm_100a kernels need on
// top: fire-and-forget `red` (no return value, so no NVLink round trip), L2-only
// loads for peer-written staging memory, 16/32-byte vector moves, and a wait
// helper that gives up after a wall-clock limit instead of spinning forever.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace pplx {
namespace ptx {

// ---------------------------------------------------------------- flags ----

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t ld_volatile(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Stores and reductions through an NVLink multicast mapping: the NVSwitch applies them to the
// same offset of every GPU bound to the multicast object.
__device__ __forceinline__ void multimem_st_relaxed_sys(void* mc, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

__device__ __forceinline__ void multimem_red_add_release_sys(void* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

__device__ __forceinline__ void multimem_st_v4(void* mc, const int4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
               "f"(__int_as_float(v.x)), "f"(__int_as_float(v.y)), "f"(__int_as_float(v.z)),
               "f"(__int_as_float(v.w))
               : "memory");
}

__device__ __forceinline__ void st_volatile(uint32_t* p, uint32_t v) {
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Release-add without a return value: the issuing thread does not wait for the
// remote memory to answer.
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void red_add_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;"
               : "=r"(old)
               : "l"(p), "r"(v)
               : "memory");
  return old;
}

__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}

__device__ __forceinline__ void fence_acq_rel_gpu() {
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
}

// Orders generic-proxy accesses (plain ld/st, including a peer's stores that an
// acquire made visible) before later async-proxy accesses (TMA, tcgen05 reads
// of shared memory).
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------- payload ----

// 16-byte load that is cached in L2 only.  Staging memory is rewritten by peers
// on every iteration, so a line left in L1 by the previous iteration must never
// satisfy the load.
__device__ __forceinline__ int4 ld_cg_v4(const void* p) {
  int4 v;
  asm volatile("ld.global.cg.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// 16-byte read-only load through the non-coherent path (inputs that no one
// writes while the kernel runs: user activations, expert outputs).
__device__ __forceinline__ int4 ld_nc_v4(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st_v4(void* p, const int4& v) {
  asm volatile("st.global.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Streaming 16-byte store for local outputs that this kernel does not read back.
__device__ __forceinline__ void st_cs_v4(void* p, const int4& v) {
  asm volatile("st.global.cs.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Warp-wide copy of `nvec` 16-byte vectors.  Loads are issued in batches of
// kBatch before the first store of the batch, so a lane keeps that many requests
// in flight instead of paying one memory latency per vector.
enum class LoadKind { kNonCoherent, kL2Only };

template <LoadKind K, int kBatch = 8>
__device__ __forceinline__ void warp_copy_v4(void* dst, const void* src, int nvec, int lane) {
  uint8_t* d = static_cast<uint8_t*>(dst);
  const uint8_t* s = static_cast<const uint8_t*>(src);
  for (int v0 = lane; v0 < nvec; v0 += 32 * kBatch) {
    int4 r[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) {
        if constexpr (K == LoadKind::kNonCoherent) r[u] = ld_nc_v4(s + (static_cast<size_t>(v) << 4));
        else r[u] = ld_cg_v4(s + (static_cast<size_t>(v) << 4));
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) st_v4(d + (static_cast<size_t>(v) << 4), r[u]);
    }
  }
}

// The same copy with the stores going through a multicast mapping: every rank bound to it
// receives the vectors at the same offset.
template <int kBatch = 8>
__device__ __forceinline__ void warp_copy_v4_multicast(void* dst_mc, const void* src, int nvec,
                                                       int lane) {
  uint8_t* d = static_cast<uint8_t*>(dst_mc);
  const uint8_t* s = static_cast<const uint8_t*>(src);
  for (int v0 = lane; v0 < nvec; v0 += 32 * kBatch) {
    int4 r[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) r[u] = ld_nc_v4(s + (static_cast<size_t>(v) << 4));
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int v = v0 + 32 * u;
      if (v < nvec) multimem_st_v4(d + (static_cast<size_t>(v) << 4), r[u]);
    }
  }
}

// Hint: bring the 128-byte line at `p` into L2.
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void nanosleep(uint32_t ns) {
  asm volatile("nanosleep.u32 %0;" ::"r"(ns));
}

}  // namespace ptx
}  // namespace pplx
