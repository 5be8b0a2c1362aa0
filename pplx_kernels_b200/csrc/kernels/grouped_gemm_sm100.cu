// Grouped expert GEMM for sm_100a: for every local expert e with counts[e] rows,
//   out[e, :counts[e], :] = act(x[e, :counts[e], :] @ w[e]^T)
// with bf16 operands, fp32 accumulation in tensor memory and a bf16 result.
// `act` is the identity, or SwiGLU when w[e] stacks a gate and an up projection
// ([2 * I, K]) and the result has I columns: silu(x @ gate^T) * (x @ up^T).
//
// The reference contains no GEMM; this kernel serves the fused MoE layer that
// goes beyond it.  Design (one CTA per SM, persistent over tiles):
//
//   warp 0      TMA producer: cp.async.bulk.tensor tile loads of x and w into a
//               ring of 128-byte-swizzled shared-memory stages (no multicast)
//   warp 1      one elected thread issues tcgen05.mma (M=128, N=256, K=16 per
//               instruction) into one of two 256-column accumulators in tensor
//               memory, and tcgen05.commit to hand stages and accumulators on
//   warp 2      allocates / frees the 512 tensor-memory columns
//   warps 4-7   epilogue: tcgen05.ld of the finished accumulator, activation,
//               bf16 conversion, masked 16-byte global stores; overlaps with the
//               MMAs of the next tile through the second accumulator
//
// Tiles are (expert, 256-column block, 128-row block) with the row block varying
// fastest, so CTAs that run at the same time share a weight tile in L2.  The
// row counts are read on the device, so the launch is graph-capturable and does
// no work for empty experts.
//
// Every mbarrier wait is bounded: when one runs out the CTA raises a shared
// abort flag, all roles leave their loops, in-flight TMA loads are drained,
// tensor memory is freed and the kernel returns with *status = 1.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../core/device_utils.cuh"
#include "../core/tcgen05.cuh"
#include "../core/utils.h"
#include "grouped_gemm.h"

namespace pplx {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kStages = 4;
constexpr int kThreads = 256;
constexpr int kTmemCols = 512;
constexpr uint32_t kABytes = kBlockM * kBlockK * 2;  // 16 KiB
constexpr uint32_t kBBytes = kBlockN * kBlockK * 2;  // 32 KiB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint64_t kWaitLimitNs = 2000000000ull;     // 2 s per wait
constexpr int kMaxExperts = 1024;

struct SharedControl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t total_tiles;
  uint32_t pad;
};

struct TileCoord {
  int expert;
  int m_blk;
  int n_blk;
  int rows;  // valid rows of the expert
};

// tile_start[e] = first tile of expert e; tiles of one expert are ordered
// (n_blk, m_blk) with m_blk fastest.
__device__ __forceinline__ TileCoord locate_tile(const uint32_t* tile_start,
                                                 const int32_t* __restrict__ counts, int E,
                                                 int capacity, uint32_t t) {
  TileCoord c;
  c.expert = find_group(tile_start, E, t);
  c.rows = min(max(counts[c.expert], 0), capacity);
  const int m_tiles = ceil_div<int>(c.rows, kBlockM);
  const uint32_t rem = t - tile_start[c.expert];
  c.n_blk = static_cast<int>(rem / m_tiles);
  c.m_blk = static_cast<int>(rem - static_cast<uint32_t>(c.n_blk) * m_tiles);
  return c;
}

__device__ __forceinline__ float silu(float v) { return v / (1.0f + __expf(-v)); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
    grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_b, const GroupedGemmArgs g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // Stage ring first (1024-byte aligned tiles), control block and tile table after.
  uint8_t* stages = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  SharedControl* ctl = reinterpret_cast<SharedControl*>(stages + kStages * kStageBytes);
  uint32_t* tile_start = reinterpret_cast<uint32_t*>(ctl + 1);  // [E + 1]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  // Output columns per tile and number of column blocks.
  const int out_cols_per_tile = SWIGLU ? kBlockN / 2 : kBlockN;
  const int n_blocks = ceil_div<int>(g.n_out, out_cols_per_tile);
  const int num_kb = ceil_div<int>(g.k, kBlockK);

  // ---- set-up ---------------------------------------------------------------
  for (int e = tid; e < g.num_experts; e += blockDim.x) {
    const int rows = min(max(g.counts[e], 0), g.rows_per_expert);
    tile_start[e] = static_cast<uint32_t>(ceil_div<int>(rows, kBlockM) * n_blocks);
  }
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&ctl->full[s], 1);
      tc::mbar_init(&ctl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&ctl->tmem_full[b], 1);
      tc::mbar_init(&ctl->tmem_empty[b], 4);
    }
    ctl->abort_flag = 0;
    tc::fence_mbar_init();
    tc::tma_prefetch_desc(&tmap_a);
    tc::tma_prefetch_desc(&tmap_b);
  }
  __syncthreads();
  if (warp == 0) warp_exclusive_scan_smem(tile_start, g.num_experts, lane, true);
  if (warp == 2) {
    tc::tmem_alloc(&ctl->tmem_base, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t total_tiles = tile_start[g.num_experts];

  // ---- roles ----------------------------------------------------------------
  if (warp == 0) {
    if (tc::elect_one()) {
      uint32_t stage = 0, phase = 0;
      uint32_t pending = 0;        // stages that have been filled at least once
      uint32_t pending_phase = 0;  // parity of the phase each stage was last filled in
      bool ok = true;
      for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord c = locate_tile(tile_start, g.counts, g.num_experts, g.rows_per_expert, t);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = tc::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag, kWaitLimitNs);
          if (!ok) break;
          uint8_t* a_dst = stages + stage * kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          tc::mbar_arrive_expect_tx(&ctl->full[stage], kStageBytes);
          pending |= 1u << stage;
          pending_phase = (pending_phase & ~(1u << stage)) | (phase << stage);
          tc::tma_load_3d(a_dst, &tmap_a, &ctl->full[stage], kb * kBlockK, c.m_blk * kBlockM,
                          c.expert);
          if constexpr (SWIGLU) {
            const int row = c.n_blk * (kBlockN / 2);
            tc::tma_load_3d(b_dst, &tmap_b, &ctl->full[stage], kb * kBlockK, row, c.expert);
            tc::tma_load_3d(b_dst + kBBytes / 2, &tmap_b, &ctl->full[stage], kb * kBlockK,
                            g.n_out + row, c.expert);
          } else {
            const int row = c.n_blk * kBlockN;
            tc::tma_load_3d(b_dst, &tmap_b, &ctl->full[stage], kb * kBlockK, row, c.expert);
            tc::tma_load_3d(b_dst + kBBytes / 2, &tmap_b, &ctl->full[stage], kb * kBlockK,
                            row + kBlockN / 2, c.expert);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag != 0u) {
        // Give the loads already issued a bounded time to land before the CTA
        // leaves: their destination is this CTA's shared memory.
        uint64_t t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (int s = 0; s < kStages; ++s) {
          if (!((pending >> s) & 1u)) continue;
          while (!tc::mbar_try_wait(&ctl->full[s], (pending_phase >> s) & 1u)) {
            uint64_t t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > 100000000ull) break;  // 100 ms in total
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (tc::elect_one()) {
      const uint32_t idesc = tc::make_instr_desc(1u, kBlockM, kBlockN);
      uint32_t stage = 0, phase = 0;
      uint32_t local = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
        const uint32_t buf = local & 1u;
        const uint32_t use = local >> 1;  // how often this accumulator was used before
        ok = tc::mbar_wait(&ctl->tmem_empty[buf], (use & 1u) ^ 1u, abort_flag, kWaitLimitNs);
        if (!ok) break;
        tc::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * kBlockN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = tc::mbar_wait(&ctl->full[stage], phase, abort_flag, kWaitLimitNs);
          if (!ok) break;
          tc::tc_fence_after_sync();
          const uint8_t* a_src = stages + stage * kStageBytes;
          const uint64_t a_desc = tc::make_smem_desc_sw128(a_src);
          const uint64_t b_desc = tc::make_smem_desc_sw128(a_src + kABytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            tc::mma_f16_ss(tmem_d, tc::advance_smem_desc(a_desc, k * kUmmaK * 2),
                           tc::advance_smem_desc(b_desc, k * kUmmaK * 2), idesc,
                           (kb | k) != 0);
          }
          tc::mma_commit(&ctl->empty[stage]);  // stage reusable once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc::mma_commit(&ctl->tmem_full[buf]);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    const int ew = warp - 4;  // lanes [32 * ew, 32 * ew + 32) of tensor memory
    uint32_t local = 0;
    bool ok = true;
    __nv_bfloat16* out = g.out;
    for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
      const TileCoord c = locate_tile(tile_start, g.counts, g.num_experts, g.rows_per_expert, t);
      const uint32_t buf = local & 1u;
      const uint32_t use = local >> 1;
      ok = tc::mbar_wait(&ctl->tmem_full[buf], use & 1u, abort_flag, kWaitLimitNs);
      if (!ok) break;
      tc::tc_fence_after_sync();
      const int row = c.m_blk * kBlockM + ew * 32 + lane;
      const bool row_ok = row < c.rows;
      __nv_bfloat16* out_row = out + static_cast<int64_t>(c.expert) * g.out_stride_e +
                               static_cast<int64_t>(row) * g.out_stride_row;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + buf * kBlockN;
      const int col0 = c.n_blk * out_cols_per_tile;
#pragma unroll 1
      for (int chunk = 0; chunk < out_cols_per_tile / 32; ++chunk) {
        uint32_t acc[32];
        uint32_t packed[16];
        tc::tmem_ld_32x32(taddr + chunk * 32, acc);
        if constexpr (SWIGLU) {
          uint32_t up[32];
          tc::tmem_ld_32x32(taddr + kBlockN / 2 + chunk * 32, up);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g0 = __uint_as_float(acc[2 * j]), g1 = __uint_as_float(acc[2 * j + 1]);
            const float u0 = __uint_as_float(up[2 * j]), u1 = __uint_as_float(up[2 * j + 1]);
            packed[j] = pack_bf16(silu(g0) * u0, silu(g1) * u1);
          }
        } else {
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            packed[j] = pack_bf16(__uint_as_float(acc[2 * j]), __uint_as_float(acc[2 * j + 1]));
          }
        }
        if (row_ok) {
          const int col = col0 + chunk * 32;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col + v * 8 + 8 <= g.n_out) {
              int4 q;
              q.x = packed[4 * v];
              q.y = packed[4 * v + 1];
              q.z = packed[4 * v + 2];
              q.w = packed[4 * v + 3];
              *reinterpret_cast<int4*>(out_row + col + v * 8) = q;
            }
          }
        }
      }
      // Accumulator drained: hand it back to the MMA warp.
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&ctl->tmem_empty[buf]);
    }
  }

  // ---- teardown -------------------------------------------------------------
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0 && ctl->abort_flag != 0u && g.status != nullptr) *g.status = 1u;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    PPLX_CHECK(q == cudaDriverEntryPointSuccess && p != nullptr,
               "cuTensorMapEncodeTiled is not available in this driver");
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// [experts, rows, k] bf16 with k contiguous; tiles of 64 x 128 x 1, 128-byte swizzle,
// out-of-range elements read as zero.
CUtensorMap make_operand_map(const void* base, int64_t experts, int64_t rows, int64_t k,
                             int64_t stride_row_elems, int64_t stride_expert_elems) {
  PPLX_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0, "operand base must be 16-byte aligned");
  PPLX_CHECK((stride_row_elems * 2) % 16 == 0 && (stride_expert_elems * 2) % 16 == 0,
             "operand strides must be multiples of 16 bytes (8 bf16 elements)");
  CUtensorMap map;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(experts)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(stride_row_elems) * 2,
                                 static_cast<cuuint64_t>(stride_expert_elems) * 2};
  const cuuint32_t box[3] = {kBlockK, 128, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = encode_tiled()(
      &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PPLX_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code " << static_cast<int>(r));
  return map;
}

size_t smem_bytes(int num_experts) {
  return 1024 + kStages * kStageBytes + sizeof(SharedControl) +
         sizeof(uint32_t) * (static_cast<size_t>(num_experts) + 1);
}

}  // namespace

void launch_grouped_gemm(const GroupedGemmCall& c, cudaStream_t stream) {
  PPLX_CHECK(c.num_experts > 0 && c.num_experts <= kMaxExperts, "num_experts out of range");
  PPLX_CHECK(c.k > 0 && c.k % 8 == 0, "K must be a positive multiple of 8");
  PPLX_CHECK(c.n_out > 0 && c.n_out % 8 == 0, "the output width must be a positive multiple of 8");
  PPLX_CHECK(!c.swiglu || c.n_out % (kBlockN / 2) == 0,
             "SwiGLU needs an intermediate size that is a multiple of 128");
  PPLX_CHECK(reinterpret_cast<uintptr_t>(c.out) % 16 == 0 && c.out_stride_row % 8 == 0 &&
                 c.out_stride_e % 8 == 0,
             "the output must be 16-byte aligned");
  const int64_t w_rows = c.swiglu ? 2 * static_cast<int64_t>(c.n_out) : c.n_out;
  const CUtensorMap tmap_a = make_operand_map(c.x, c.num_experts, c.rows_per_expert, c.k,
                                              c.x_stride_row, c.x_stride_e);
  const CUtensorMap tmap_b =
      make_operand_map(c.w, c.num_experts, w_rows, c.k, c.w_stride_row, c.w_stride_e);

  GroupedGemmArgs g{};
  g.counts = c.counts;
  g.out = static_cast<__nv_bfloat16*>(c.out);
  g.out_stride_e = c.out_stride_e;
  g.out_stride_row = c.out_stride_row;
  g.status = c.status;
  g.num_experts = c.num_experts;
  g.rows_per_expert = c.rows_per_expert;
  g.n_out = c.n_out;
  g.k = c.k;

  const size_t smem = smem_bytes(c.num_experts);
  const int grid = c.num_sms > 0 ? c.num_sms : get_sm_count();
  if (c.swiglu) {
    CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_kernel<true>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem_bytes(kMaxExperts))));
    grouped_gemm_kernel<true><<<grid, kThreads, smem, stream>>>(tmap_a, tmap_b, g);
  } else {
    CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_kernel<false>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem_bytes(kMaxExperts))));
    grouped_gemm_kernel<false><<<grid, kThreads, smem, stream>>>(tmap_a, tmap_b, g);
  }
  CUDA_CHECK(cudaGetLastError());
}

}  // namespace pplx
