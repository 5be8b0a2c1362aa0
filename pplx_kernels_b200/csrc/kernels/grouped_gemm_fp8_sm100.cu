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
// With power-of-two scales (`pow2_scales`) the tensor cores apply them themselves
// (kind::mxf8f6f4.block_scale): warp 3 turns the fp32 scales of each K block into E8M0 bytes in
// the layout tcgen05.cp takes, the MMA thread copies them into tensor memory in front of the
// block's four MMAs, the whole K range accumulates in ONE tensor-memory accumulator, and the
// fold warps only read the finished tile (and free the accumulator before they convert and
// store, so that the next tile's MMAs run under the epilogue).
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
#include "../core/wait.cuh"
#include "a2a_device.cuh"
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
constexpr uint32_t kSfAtomBytes = 512;
constexpr uint32_t kSfStageBytes = 3 * kSfAtomBytes;
constexpr uint32_t kSfaCol = 256;  // tensor-memory columns of the scales, behind the accumulator
constexpr uint32_t kSfbCol = 260;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr int kMaxExperts = 1024;

struct SharedControl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t part_full[2];   // scratch accumulator holds a finished K block
  uint64_t part_empty[2];  // scratch accumulator may be overwritten
  uint64_t acc_full;       // hardware-scaled form: the tile's accumulator is complete
  uint64_t acc_empty;      //                       ... has been read out by all fold warps
  uint32_t tmem_base;
  uint32_t abort_flag;
  float row_amax[2][kBlockM];  // SwiGLU epilogue: per-row maxima of the two column halves
  uint32_t sig_token[kBlockM];  // peer-storing epilogue: token of each tile row
  uint32_t sig_group[kBlockM];  //                        first rank of the token's DP group
  // Hardware-scaled form: per stage the E8M0 scales of the K block in the layout tcgen05.cp
  // takes (32 rows of 16 bytes per 128 rows or columns): A rows, B columns 0-127, 128-255.
  alignas(128) uint8_t sf[kStages][kSfStageBytes];
};

constexpr uint32_t kNoSignalFp8 = 0xffffffffu;

// Staging of the peer-storing epilogue: per fold warp 32 rows x (64 B + 16 B pad).
constexpr int kFp8StageRowBytes = 80;
constexpr uint32_t kSignalQueue = 512;
struct Fp8PeerStage {
  uint8_t rows[8][32][kFp8StageRowBytes];
  unsigned long long row_off[kBlockM];  // arena offset of each tile row's combine slot
  uint32_t q_token[kSignalQueue];        // queued arrival adds: token ...
  uint32_t q_group_units[kSignalQueue];  // ... first rank of its DP group | columns << 8
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

__device__ __forceinline__ Fp8Tile locate(const uint32_t* tile_start, const uint32_t* rows_of,
                                          int num_experts, uint32_t t) {
  Fp8Tile c;
  c.expert = find_group(tile_start, num_experts, t);
  c.rows = static_cast<int>(rows_of[c.expert]);
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

namespace {

constexpr size_t kMaxSrcEntriesFp8 = 2048;

size_t fp8_smem_bytes(size_t experts, size_t src_entries, bool to_peers) {
  return 1024 + kStages * kStageBytes + sizeof(SharedControl) +
         sizeof(uint32_t) * (3 * experts + 1 + src_entries) +
         (to_peers ? sizeof(Fp8PeerStage) + 16 : 0);
}

void check_fp8_call(const Fp8GemmCall& c, bool need_x, bool need_out) {
  PPLX_CHECK(c.num_experts > 0 && c.num_experts <= kMaxExperts, "num_experts out of range");
  PPLX_CHECK(c.k > 0 && c.k % 16 == 0, "K must be a positive multiple of 16");
  PPLX_CHECK(c.n_out > 0 && c.n_out % 16 == 0, "the output width must be a multiple of 16");
  PPLX_CHECK(!c.swiglu_quant || c.n_out % 128 == 0,
             "the SwiGLU + quantise epilogue needs an intermediate size that is a multiple of 128");
  PPLX_CHECK(c.w && c.sw, "missing weight tensor");
  PPLX_CHECK(!need_x || (c.x && c.sa && c.counts), "missing activation tensor");
  PPLX_CHECK(!need_out || c.out, "missing output tensor");
  PPLX_CHECK(!c.swiglu_quant || c.out_scale != nullptr, "out_scale is required");
  PPLX_CHECK(reinterpret_cast<uintptr_t>(c.out) % 16 == 0, "the output must be 16-byte aligned");
}

Fp8GemmArgs fp8_args(const Fp8GemmCall& c) {
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
  return g;
}

template <bool kSwiGLUQuant, bool kFromStaging, bool kToPeers, bool kPow2 = false>
void launch_fp8(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const Fp8GemmArgs& g,
                int num_sms, cudaStream_t stream) {
  auto* kernel = grouped_gemm_fp8_kernel<kSwiGLUQuant, kFromStaging, kToPeers, kPow2>;
  const size_t src_entries =
      (kFromStaging && g.src_table != 0) ? static_cast<size_t>(g.num_experts) * g.a2a.world : 0;
  const size_t smem = fp8_smem_bytes(g.num_experts, src_entries, kToPeers);
  PPLX_CHECK(smem <= 227 * 1024, "the tile tables of " << g.num_experts << " experts need "
                                                       << smem << " bytes of shared memory");
  CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
  const int grid = num_sms > 0 ? num_sms : get_sm_count();
  kernel<<<grid, kThreads, smem, stream>>>(tmap_a, tmap_b, g);
  CUDA_CHECK(cudaGetLastError());
}

}  // namespace

void launch_grouped_gemm_fp8(const Fp8GemmCall& c, cudaStream_t stream) {
  check_fp8_call(c, true, true);
  const int64_t w_rows = c.swiglu_quant ? 2 * static_cast<int64_t>(c.n_out) : c.n_out;
  const CUtensorMap tmap_a =
      make_byte_map(c.x, c.num_experts, c.rows_per_expert, c.k, c.x_stride_row, c.x_stride_e);
  const CUtensorMap tmap_b =
      make_byte_map(c.w, c.num_experts, w_rows, c.k, c.w_stride_row, c.w_stride_e);
  const Fp8GemmArgs g = fp8_args(c);
  if (c.pow2_scales) {
    if (c.swiglu_quant) launch_fp8<true, false, false, true>(tmap_a, tmap_b, g, c.num_sms, stream);
    else launch_fp8<false, false, false, true>(tmap_a, tmap_b, g, c.num_sms, stream);
  } else if (c.swiglu_quant) {
    launch_fp8<true, false, false>(tmap_a, tmap_b, g, c.num_sms, stream);
  } else {
    launch_fp8<false, false, false>(tmap_a, tmap_b, g, c.num_sms, stream);
  }
}

void launch_gemm_fp8_from_staging(const Fp8GemmCall& c, const A2AParams& p,
                                  int32_t* out_num_tokens, cudaStream_t stream) {
  check_fp8_call(c, false, true);
  PPLX_CHECK(c.swiglu_quant, "the staging-fed fp8 GEMM is the SwiGLU up projection");
  PPLX_CHECK(p.hidden_bytes == p.hidden_dim && p.scale_bytes == ceil_div(p.hidden_dim, 128) * 4,
             "the staging-fed fp8 GEMM needs an object created for a 1-byte payload with one "
             "fp32 scale per 128 columns");
  PPLX_CHECK(c.k == p.hidden_dim && c.num_experts == p.nle && c.rows_per_expert >= p.cap,
             "shape mismatch between the GEMM and the all-to-all");
  // A: [1][world * region_slots][hidden] e4m3 view of this rank's packed staging.
  const int64_t slots = static_cast<int64_t>(p.world) * p.region_slots;
  const CUtensorMap tmap_a = make_byte_map(p.peer[p.rank] + p.off_disp_stage, 1, slots,
                                           p.hidden_dim, p.slot_bytes, slots * p.slot_bytes);
  const CUtensorMap tmap_b = make_byte_map(c.w, c.num_experts, 2 * static_cast<int64_t>(c.n_out),
                                           c.k, c.w_stride_row, c.w_stride_e);
  Fp8GemmArgs g = fp8_args(c);
  g.out_num_tokens = out_num_tokens;
  g.a2a = p;
  g.src_table = static_cast<size_t>(p.nle) * p.world <= kMaxSrcEntriesFp8 ? 1 : 0;
  if (c.pow2_scales) launch_fp8<true, true, false, true>(tmap_a, tmap_b, g, c.num_sms, stream);
  else launch_fp8<true, true, false>(tmap_a, tmap_b, g, c.num_sms, stream);
}

void launch_gemm_fp8_to_peers(const Fp8GemmCall& c, const A2AParams& p, cudaStream_t stream) {
  check_fp8_call(c, true, false);
  PPLX_CHECK(!c.swiglu_quant, "the peer-storing fp8 GEMM is the plain down projection");
  PPLX_CHECK(c.n_out == p.hidden_dim && c.num_experts == p.nle && c.rows_per_expert >= p.cap,
             "shape mismatch between the GEMM and the all-to-all");
  PPLX_CHECK(c.counts == reinterpret_cast<const int32_t*>(p.recv_count),
             "counts must be the all-to-all's received-row counts");
  PPLX_CHECK(p.dp_size <= 8, "at most 8 replicas per DP group");
  const CUtensorMap tmap_a =
      make_byte_map(c.x, c.num_experts, c.rows_per_expert, c.k, c.x_stride_row, c.x_stride_e);
  const CUtensorMap tmap_b =
      make_byte_map(c.w, c.num_experts, c.n_out, c.k, c.w_stride_row, c.w_stride_e);
  Fp8GemmArgs g = fp8_args(c);
  g.out = nullptr;
  g.a2a = p;
  if (c.pow2_scales) launch_fp8<false, false, true, true>(tmap_a, tmap_b, g, c.num_sms, stream);
  else launch_fp8<false, false, true>(tmap_a, tmap_b, g, c.num_sms, stream);
}

}  // namespace pplx
