// Grouped expert GEMM (tcgen05 / tensor memory / TMA) -- host interface.
// No counterpart in the reference, which has no GEMM.
#pragma once

#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "a2a_params.h"

namespace pplx {

constexpr int kNumTileWidths = 5;

// Device-side arguments (the tensor maps travel as separate kernel parameters).
struct GroupedGemmArgs {
  const int32_t* counts;   // [num_experts] valid rows per expert
  __nv_bfloat16* out;      // [num_experts][rows_per_expert][n_out]
  int64_t out_stride_e;    // elements
  int64_t out_stride_row;  // elements
  uint32_t* status;        // optional device word, set to 1 if a wait ran out
  int num_experts;
  int rows_per_expert;     // capacity of x / out per expert
  int n_out;               // output columns (the intermediate size for SwiGLU)
  int k;
  int widths[kNumTileWidths];  // candidate weight rows per B half (the tile is twice as wide
                               // in columns); 0 = not available.  Chosen on the device.
  // Only read by the kernels fused with the all-to-all:
  int32_t* out_num_tokens;          // optional [nle]: per-expert totals for the caller
  int src_table;                    // staging-fed form: keep rows per (expert, source) in
                                    // shared memory (set by the launcher when it fits)
  A2AParams a2a;
};

// Host-side description of one launch.  Strides are in bf16 elements; the
// innermost (K) stride of x and w is 1.
struct GroupedGemmCall {
  const void* x = nullptr;   // [num_experts][rows_per_expert][k]
  int64_t x_stride_e = 0;
  int64_t x_stride_row = 0;
  const void* w = nullptr;   // [num_experts][n_out or 2 * n_out][k]
  int64_t w_stride_e = 0;
  int64_t w_stride_row = 0;
  const int32_t* counts = nullptr;
  void* out = nullptr;
  int64_t out_stride_e = 0;
  int64_t out_stride_row = 0;
  uint32_t* status = nullptr;
  int num_experts = 0;
  int rows_per_expert = 0;
  int n_out = 0;
  int k = 0;
  bool swiglu = false;
  int num_sms = 0;           // 0 = all
  int half_n = 0;            // 0 = choose; else weight rows per B half (multiple of 8, 64..128)
  int64_t expected_total_rows = 0;  // hint for the tile-width choice; 0 = capacity
  int cta_pair = -1;         // -1 = choose, 0 = one CTA per 128-row tile, 1 = CTA pair per
                             // 256-row tile (tcgen05 cta_group::2)
};

// out[e, :counts[e]] = act(x[e, :counts[e]] @ w[e]^T); rows beyond counts[e] are untouched.
void launch_grouped_gemm(const GroupedGemmCall& call, cudaStream_t stream);

// First expert GEMM of the fused MoE layer.  Takes the place of the dispatch
// receive phase: A is read from the dispatch staging arena of `p` as peers fill
// it (bf16 payload without scales), out[le] receives SwiGLU(x @ w[le]^T) for the
// rows of local expert le, `out_num_tokens` (optional) the per-expert totals.
// call.x / call.counts are ignored; call.k must equal the hidden size of `p`.
void launch_gemm_from_staging(const GroupedGemmCall& call, const A2AParams& p,
                              int32_t* out_num_tokens, cudaStream_t stream);

// Second expert GEMM of the fused MoE layer.  Takes the place of the combine send
// phase: every output row x[le, r] @ w[le]^T goes to the combine staging of the
// token's home rank(s); call.out is ignored, call.counts must be p.recv_count and
// call.n_out the hidden size of `p`.  Every column block adds its columns to the tokens'
// arrival counters, so any tile width can be chosen.
void launch_gemm_to_peers(const GroupedGemmCall& call, const A2AParams& p, cudaStream_t stream);

}  // namespace pplx

namespace pplx {

// Block-scaled fp8 (e4m3) grouped GEMM.  Payload strides in bytes (= elements), scale
// strides in floats; the innermost strides are 1.  sa: one scale per row and 128 columns
// of K; sw: one per 128 x 128 block of w.
struct Fp8GemmCall {
  const void* x = nullptr;      // e4m3 [E][rows][k]
  int64_t x_stride_e = 0, x_stride_row = 0;
  const float* sa = nullptr;    // [E][rows][ceil(k / 128)]
  int64_t sa_stride_e = 0, sa_stride_row = 0;
  const void* w = nullptr;      // e4m3 [E][n_out or 2 * n_out][k]
  int64_t w_stride_e = 0, w_stride_row = 0;
  const float* sw = nullptr;    // [E][ceil(w rows / 128)][ceil(k / 128)]
  int64_t sw_stride_e = 0, sw_stride_row = 0;
  const int32_t* counts = nullptr;
  void* out = nullptr;          // bf16 [E][rows][n_out], or e4m3 with swiglu_quant
  int64_t out_stride_e = 0, out_stride_row = 0;  // elements
  float* out_scale = nullptr;   // swiglu_quant: [E][rows][n_out / 128]
  int64_t os_stride_e = 0, os_stride_row = 0;
  uint32_t* status = nullptr;   // optional device word: 1 a wait ran out, 2 (pow2_scales) a scale
                                // was not a power of two
  int num_experts = 0, rows_per_expert = 0, n_out = 0, k = 0;
  bool swiglu_quant = false;    // w = [gate; up]; result silu(gate) * up quantised to e4m3
  // Every scale in sa and sw is a power of two (the caller's promise; mantissa bits would be
  // ignored): the tensor cores apply them (kind::mxf8f6f4.block_scale) instead of the CUDA
  // cores, and the swiglu_quant epilogue emits power-of-two scales in turn.
  bool pow2_scales = false;
  int num_sms = 0;
};

void launch_grouped_gemm_fp8(const Fp8GemmCall& call, cudaStream_t stream);

// The fp8 forms of the two expert GEMMs of the fused MoE layer (see the bf16 functions
// above for the protocol).  from_staging: A and its scales are read from the dispatch
// staging arena after a packed, quantising send (call.x / sa / counts are ignored); the
// result is the SwiGLU-ed, re-quantised intermediate.  to_peers: the bf16 rows of the down
// projection are stored to the tokens' home ranks (call.out is ignored, call.counts must be
// p.recv_count).
void launch_gemm_fp8_from_staging(const Fp8GemmCall& call, const A2AParams& p,
                                  int32_t* out_num_tokens, cudaStream_t stream);
void launch_gemm_fp8_to_peers(const Fp8GemmCall& call, const A2AParams& p, cudaStream_t stream);

}  // namespace pplx
