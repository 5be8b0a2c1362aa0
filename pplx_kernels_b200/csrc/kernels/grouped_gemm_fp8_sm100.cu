// Block-scaled fp8 grouped expert GEMM for sm_100a (tcgen05 kind::f8f6f4).
//
//   out[e, r, :] = act( sum_kb  sa[e, r, kb] * sw[e, n / 128, kb] *
//                               (xq[e, r, kb-th 128 columns] . wq[e, n, kb-th 128 columns]) )
//
// xq / wq are e4m3, sa is one fp32 scale per row and 128 columns of K (what
// `dispatch_quant` delivers), sw one fp32 scale per 128 x 128 block of the weight
// (the DeepSeek-V3 / Qwen3 fp8 checkpoint format).  The reference has no GEMM;
// this kernel is the fp8 arm of the MoE layer that goes beyond it.
//
// fp32 scales per 128 columns are not the hardware's block-scale format, so each
// 128-wide K block is multiplied on the tensor cores into one of two scratch
// accumulators in tensor memory (four K = 32 MMAs, M = 128, N = 256) and eight
// epilogue warps fold it, times the two scales, into the running result that
// they keep in REGISTERS: warps 4-7 own output columns [0, 64) of each half of the
// tile, warps 8-11 columns [64, 128), so a thread holds 128 fp32 accumulators and
// only reads tensor memory (tcgen05.ld), while the MMAs of the next K block fill
// the other scratch accumulator.
//
// Epilogues:  kBf16   plain down projection, bf16 result, 256 columns per tile
//             kSwiGLUQuant   w stacks gate and up rows; the tile is 128 gate + 128 up
//                     rows, the result silu(gate) * up is 128 columns = exactly one
//                     scale block, so it is quantised right here to e4m3 + one fp32
//                     scale per row and tile -- the input format of the next GEMM.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warp 2 tensor-memory allocation,
// warps 4-11 scale-and-accumulate + epilogue.  All waits are bounded; on expiry the
// CTA drains, frees its tensor memory and reports through *status.
#include <algorithm>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../core/device_utils.cuh"
#include "../core/ptx.cuh"
#include "../core/tcgen05.cuh"
#include "../core/utils.h"
#include "grouped_gemm.h"

namespace pplx {
namespace {

constexpr int kBlockM = 128;
constexpr int kTileN = 256;        // weight rows per tile (UMMA N)
constexpr int kBlockKBytes = 128;  // 128 e4m3 values = one swizzle row = one scale block
constexpr int kUmmaKBytes = 32;
constexpr int kStages = 4;
constexpr int kThreads = 384;
constexpr int kTmemCols = 512;     // two scratch accumulators of 256 columns
constexpr uint32_t kABytes = kBlockM * kBlockKBytes;
constexpr uint32_t kBBytes = kTileN * kBlockKBytes;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr int kMaxExperts = 1024;

struct SharedControl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t part_full[2];   // scratch accumulator holds a finished K block
  uint64_t part_empty[2];  // scratch accumulator may be overwritten
  uint32_t tmem_base;
  uint32_t abort_flag;
  float row_amax[2][kBlockM];  // SwiGLU epilogue: per-row maxima of the two column halves
};

__device__ __forceinline__ float silu(float v) { return v / (1.0f + __expf(-v)); }

// 32 lanes x 16 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

struct Fp8Tile {
  int expert, m_blk, n_blk, rows;
};

__device__ __forceinline__ Fp8Tile locate(const uint32_t* tile_start, const int32_t* counts,
                                          int num_experts, int capacity, uint32_t t) {
  Fp8Tile c;
  c.expert = find_group(tile_start, num_experts, t);
  c.rows = min(max(counts[c.expert], 0), capacity);
  const int m_tiles = ceil_div<int>(c.rows, kBlockM);
  const uint32_t rem = t - tile_start[c.expert];
  c.n_blk = static_cast<int>(rem / m_tiles);
  c.m_blk = static_cast<int>(rem - static_cast<uint32_t>(c.n_blk) * m_tiles);
  return c;
}

}  // namespace
}  // namespace pplx

#include "grouped_gemm_fp8_kernel.inl"

namespace pplx {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fp8() {
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

// [experts, rows, k] one-byte elements with k contiguous; tiles of 128 B x 128 rows x 1,
// 128-byte swizzle, out-of-range elements read as zero.
CUtensorMap make_byte_map(const void* base, int64_t experts, int64_t rows, int64_t k,
                          int64_t stride_row, int64_t stride_expert) {
  PPLX_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0 && stride_row % 16 == 0 &&
                 stride_expert % 16 == 0,
             "fp8 operands must be 16-byte aligned with strides that are multiples of 16");
  CUtensorMap map;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(experts)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(stride_row),
                                 static_cast<cuuint64_t>(stride_expert)};
  const cuuint32_t box[3] = {kBlockKBytes, 128, 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = encode_tiled_fp8()(
      &map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PPLX_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code " << static_cast<int>(r));
  return map;
}

}  // namespace

void launch_grouped_gemm_fp8(const Fp8GemmCall& c, cudaStream_t stream) {
  PPLX_CHECK(c.num_experts > 0 && c.num_experts <= kMaxExperts, "num_experts out of range");
  PPLX_CHECK(c.k > 0 && c.k % 16 == 0, "K must be a positive multiple of 16");
  PPLX_CHECK(c.n_out > 0 && c.n_out % 16 == 0, "the output width must be a multiple of 16");
  PPLX_CHECK(!c.swiglu_quant || c.n_out % 128 == 0,
             "the SwiGLU + quantise epilogue needs an intermediate size that is a multiple of 128");
  PPLX_CHECK(c.x && c.w && c.sa && c.sw && c.out && c.counts, "missing tensor");
  PPLX_CHECK(!c.swiglu_quant || c.out_scale != nullptr, "out_scale is required");
  PPLX_CHECK(reinterpret_cast<uintptr_t>(c.out) % 16 == 0, "the output must be 16-byte aligned");
  const int64_t w_rows = c.swiglu_quant ? 2 * static_cast<int64_t>(c.n_out) : c.n_out;
  const CUtensorMap tmap_a =
      make_byte_map(c.x, c.num_experts, c.rows_per_expert, c.k, c.x_stride_row, c.x_stride_e);
  const CUtensorMap tmap_b =
      make_byte_map(c.w, c.num_experts, w_rows, c.k, c.w_stride_row, c.w_stride_e);
  Fp8GemmArgs g{};
  g.counts = c.counts;
  g.sa = c.sa;
  g.sa_stride_e = c.sa_stride_e;
  g.sa_stride_row = c.sa_stride_row;
  g.sw = c.sw;
  g.sw_stride_e = c.sw_stride_e;
  g.sw_stride_row = c.sw_stride_row;
  g.out = c.out;
  g.out_stride_e = c.out_stride_e;
  g.out_stride_row = c.out_stride_row;
  g.out_scale = c.out_scale;
  g.os_stride_e = c.os_stride_e;
  g.os_stride_row = c.os_stride_row;
  g.status = c.status;
  g.num_experts = c.num_experts;
  g.rows_per_expert = c.rows_per_expert;
  g.n_out = c.n_out;
  g.k = c.k;
  const size_t smem = 1024 + kStages * kStageBytes + sizeof(SharedControl) +
                      sizeof(uint32_t) * (static_cast<size_t>(c.num_experts) + 1);
  const size_t smem_max = 1024 + kStages * kStageBytes + sizeof(SharedControl) +
                          sizeof(uint32_t) * (kMaxExperts + 1);
  const int grid = c.num_sms > 0 ? c.num_sms : get_sm_count();
  if (c.swiglu_quant) {
    CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_fp8_kernel<true>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem_max)));
    grouped_gemm_fp8_kernel<true><<<grid, kThreads, smem, stream>>>(tmap_a, tmap_b, g);
  } else {
    CUDA_CHECK(cudaFuncSetAttribute(grouped_gemm_fp8_kernel<false>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem_max)));
    grouped_gemm_fp8_kernel<false><<<grid, kThreads, smem, stream>>>(tmap_a, tmap_b, g);
  }
  CUDA_CHECK(cudaGetLastError());
}

}  // namespace pplx
