// sm_100a building blocks for tensor-core kernels: mbarriers with bounded waits,
// TMA tile loads, tensor-memory allocation, tcgen05.mma / commit / ld, and the
// shared-memory and instruction descriptors that tcgen05.mma consumes.
//
// The reference has no tensor-core code at all; this header exists for the
// grouped expert GEMM and the fused MoE kernels that go beyond it.
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

namespace pplx {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------ mbarrier ----

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Waits for the phase with the given parity to complete, for at most `limit_ns`.
// `abort_flag` is a shared-memory word that any role of the CTA sets when it
// gives up; once set, every wait returns false at its next check so that the CTA
// drains to its teardown instead of hanging.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          volatile uint32_t* abort_flag, uint64_t limit_ns) {
  for (int i = 0; i < 64; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  while (true) {
    for (int i = 0; i < 16; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag != 0u) return false;
    uint64_t t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (t1 - t0 > limit_ns) {
      *abort_flag = 1u;
      return false;
    }
  }
}

// ----------------------------------------------------------------- TMA ----

// 3-D tiled load, no multicast: global (tensor map) -> this CTA's shared memory,
// completion counted in bytes on `bar`.  crd0 is the innermost coordinate and,
// times the element size, must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar,
                                            int crd0, int crd1, int crd2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)),
        "r"(crd0), "r"(crd1), "r"(crd2)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// Variant for a CTA pair (cta_group::2): each CTA loads into its own shared memory,
// but the bytes are counted on the mbarrier of the pair's leader (even CTA rank).
// No multicast: the two CTAs load different data.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;  // clears the pair bit of a shared::cluster address

__device__ __forceinline__ void tma_load_3d_2cta(void* smem_dst, const void* tmap,
                                                 uint64_t* leader_bar, int crd0, int crd1,
                                                 int crd2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)),
        "r"(smem_u32(leader_bar) & kPeerBitMask), "r"(crd0), "r"(crd1), "r"(crd2)
      : "memory");
}

// ------------------------------------------------------------- clusters ----

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrives on the mbarrier at the same offset in the pair leader's shared memory.
__device__ __forceinline__ void mbar_arrive_on_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(
                   smem_u32(bar) & kPeerBitMask)
               : "memory");
}

// -------------------------------------------------------- tensor memory ----

// Whole-warp calls.  `ncols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_alloc_2cta(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_2cta() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------- descriptors ----

// Shared-memory operand descriptor for a K-major tile stored with the 128-byte
// swizzle that TMA produces (rows of 128 bytes, groups of 8 rows = 1024 bytes;
// the tile base must be 1024-byte aligned).  Fields: start address >> 4 in bits
// [0,14); leading byte offset (unused for swizzled K-major) in [16,30); stride
// byte offset = 1024 >> 4 in [32,46); descriptor version 1 in [46,48); layout
// type 2 (SWIZZLE_128B) in [61,64).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(const void* smem_tile) {
  const uint64_t addr = (smem_u32(smem_tile) & 0x3ffffu) >> 4;
  uint64_t desc = addr;
  desc |= static_cast<uint64_t>(1) << 16;           // LBO (ignored)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;   // SBO
  desc |= static_cast<uint64_t>(1) << 46;           // version
  desc |= static_cast<uint64_t>(2) << 61;           // SWIZZLE_128B
  return desc;
}

// Advancing along K inside the swizzle atom moves the start address by the byte
// offset (in 16-byte units).
__device__ __forceinline__ uint64_t advance_smem_desc(uint64_t desc, uint32_t bytes) {
  return desc + (bytes >> 4);
}

// Instruction descriptor for kind::f16 with fp32 accumulation, both operands
// K-major.  ab_format: 0 = f16, 1 = bf16.  For kind::f8f6f4: 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t make_instr_desc(uint32_t ab_format, int m, int n) {
  return (1u << 4)                              // accumulator format: f32
         | (ab_format << 7)                     // A format
         | (ab_format << 10)                    // B format
         | (static_cast<uint32_t>(n >> 3) << 17)
         | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---- hardware block scaling (kind::mxf8f6f4.block_scale) ----
//
// Every 32 K-elements of a row of A and of a column of B carry one power-of-two scale (E8M0:
// value 2^(byte - 127)).  The scales of one MMA sit in tensor memory: for M (or N) = 128 rows
// the byte of row r0 + 32 * r1 is byte `id` of the 32-bit cell at lane r0 (replicated in all
// four lane quarters), column base + r1; `id` (0..3) selects one of four K = 32 steps, so one
// copy serves a 128-wide K block.  tcgen05.cp brings them there from shared memory, where the
// same 128 x 4 bytes are laid out as 32 rows of 16 bytes: byte 16 * r0 + 4 * r1 + id.

// Instruction descriptor: e4m3 x e4m3, E8M0 scales, both operands K-major.
__host__ __device__ constexpr uint32_t make_instr_desc_mxf8(int m, int n, uint32_t sf_id) {
  return (sf_id << 4)                               // B scale id
         | (static_cast<uint32_t>(n >> 3) << 17)
         | (1u << 23)                               // scale format: E8M0
         | (static_cast<uint32_t>(m >> 4) << 24)
         | (sf_id << 29);                           // A scale id
}

// Descriptor of 32 rows x 16 bytes stored contiguously without swizzle (8-row core matrices of
// 128 bytes, one after the other).
__device__ __forceinline__ uint64_t make_smem_desc_rows16(const void* smem) {
  uint64_t desc = (smem_u32(smem) & 0x3ffffu) >> 4;
  desc |= static_cast<uint64_t>(128 >> 4) << 32;    // SBO: next group of 8 rows
  desc |= static_cast<uint64_t>(1) << 46;           // version
  return desc;                                      // layout type 0: no swizzle
}

// 32 rows x 128 bits of shared memory -> tensor-memory lanes 0..31 of all four lane quarters,
// four consecutive columns at `taddr`.  Issued by one thread; ordered with the tcgen05.mma
// instructions the same thread issues before and after it.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc)
               : "memory");
}

__device__ __forceinline__ void mma_mxf8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                            bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u),
        "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

// -------------------------------------------------------------- mma etc. ----

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread.
__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                           uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}

__device__ __forceinline__ void mma_f8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}

// CTA-pair MMA (M = 256 over two SMs): issued by one thread of the leader CTA; A rows
// and B rows come half from each CTA's shared memory at the descriptors' offsets.
__device__ __forceinline__ void mma_f16_ss_2cta(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate ? 1u : 0u)
      : "memory");
}

// Arrival on the mbarrier at this offset in every CTA of `cta_mask` once the pair's
// MMAs issued so far have finished.  (Multicast of a barrier arrival, not of data.)
__device__ __forceinline__ void mma_commit_2cta(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}

// Makes `bar` complete one arrival once all tcgen05.mma issued so far by this
// thread have finished (reading shared memory and writing tensor memory).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives row
// (lane base + t), columns [col, col + 32).  A warp may only touch the 32 lanes
// that start at 32 * (warp index % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace tc
}  // namespace pplx
