// Plain-data description of one rank's all-to-all state, shared by host and device.
//
// Role parity: the reference's device-side `BufferWrapper` (intranode.cuh:10-64)
// and the buffer tables of AllToAllIntraNode / AllToAllInterNode
// (intranode.h:66-88, internode.h:111-132).  The design differs:
//
//  * One symmetric arena per rank holds every region that peers touch, at the
//    same offsets on every rank, so the kernels need a single table of peer base
//    pointers.
//  * Dispatch staging is keyed by SOURCE RANK only.  A sender sorts its rows by
//    destination-local expert with a prefix sum it computes from `indices`, so
//    the region holds at most `ceil(max_tokens/dp_size) * min(topk, nle)` slots
//    instead of `nle * max_tokens`.
//  * Combine staging is keyed by (token, k): each token's top-k expert outputs
//    sit side by side at its home rank, `max_tokens * topk` rows in total rather
//    than `max_tokens * num_experts`.
//  * Counts and arrival counters exist twice, selected by the parity of a
//    device-side iteration counter.  No flag handshake is needed before a send:
//    a rank can be at most one dispatch ahead of any peer, because every rank
//    posts counts to every rank in every dispatch.
//  * A second, "packed" send mode serves the fused MoE layer: every rank first
//    posts its whole per-expert histogram to every rank, waits for everyone's,
//    and then stores each row at its final position in the destination's
//    staging, grouped by local expert and then by source.  It costs one more
//    flag round trip before the payload moves, and gives the expert GEMM dense
//    128-row tiles that it can read with TMA without any receive-side copy.
//    Arrival is counted per (local expert, source), so the GEMM can start a tile
//    as soon as the sources whose rows it covers have landed.
//  * Resets ride on the strict dispatch/combine alternation: a combine clears the
//    flag set of the dispatch before it and bumps the iteration counter.  The
//    combine's per-token arrival counters are never cleared: every combine adds
//    hidden_dim * topk to each of them (one unit per column that landed: peers for
//    live tokens, the owner itself for tokens at or beyond bound_m), so the n-th
//    combine waits for n * hidden_dim * topk modulo 2^32.
#pragma once

#include <cstddef>
#include <cstdint>

#include "../core/status.h"

namespace pplx {

constexpr int kMaxWorld = 16;

struct A2AParams {
  // geometry
  int rank;
  int world;
  int dp_size;
  int num_dp_groups;
  int num_experts;       // padded to nle * world
  int num_real_experts;  // what the caller configured (<= num_experts)
  int nle;           // experts owned by each rank
  int topk;
  int max_tokens;    // per DP group and step
  int hidden_dim;    // elements
  int hidden_bytes;  // dispatch payload bytes per token (multiple of 16)
  int scale_bytes;   // fp32 scale bytes per token (multiple of 4, may be 0)
  int trailer_off;   // round_up(hidden_bytes + scale_bytes, 16): where the trailer sits
  int slot_bytes;    // trailer_off + 16
  int region_slots;  // dispatch staging slots per source rank
  int cap;           // rows per local expert in out_expert_x / expert_y
  int debug_checks;  // non-zero: bounds checks that record instead of corrupting
  int quant_pow2;    // non-zero: the quantising sends emit power-of-two scales, and the fp8 expert
                     // GEMMs of the fused path let the tensor cores apply them
  int comb_units;    // arrival units one complete expert output row is worth: its columns
  // Flag-in-data protocol (core/ll128.cuh) for the plain dispatch and combine.
  int ll;                  // non-zero: in use
  int ll_x_lines;          // 128-byte lines that carry a dispatch row's token payload
  int ll_meta_lines;       // lines that carry its trailer and scales
  int ll_slot_bytes;       // (ll_x_lines + ll_meta_lines) * 128
  int ll_comb_slot_bytes;  // lines of one fp32 expert output row * 128
  int tiny;                // non-zero: the plain dispatch runs the decode-sized kernel

  // offsets into the symmetric arena (bytes, 256-aligned)
  size_t off_counts;        // u32 [2][world][nle]   value = count + 1, 0 = not posted
  size_t off_arrived;       // u32 [2][world]        rows landed from each source
  size_t off_comb_arrived;  // u32 [max_tokens]      running total, 16 units per expert output
  size_t off_counts_all;    // u32 [2][world][num_experts]  packed mode: every source's full
                            //                       histogram, value = count + 1
  size_t off_arrived_e;     // u32 [2][nle][world]   packed mode: rows landed per local expert
                            //                       and source rank
  size_t off_disp_stage;    // u8  [world][region_slots][slot_bytes]; in packed mode the same
                            //     memory is one array of world * region_slots slots with
                            //     rows grouped by local expert, then by source rank
  size_t off_comb_stage;    // u8  [max_tokens*topk][hidden_dim*4]
  size_t off_ll_disp_stage; // u8  [world][region_slots][ll_slot_bytes], written only as lines
  size_t off_ll_comb_stage; // u8  [max_tokens*topk][ll_comb_slot_bytes], written only as lines
  size_t off_tiny_hdr;      // u8  [2][world][ceil(max_tokens/dp_size)][128]: decode-sized dispatch,
                            //     one header line per (parity, source, token)
  size_t arena_bytes;

  uint8_t* peer[kMaxWorld];  // arena base of every rank as mapped in this process
  uint8_t* mc;  // NVLink multicast alias of the arenas (same offsets on all ranks), or nullptr
  int mc_combine;  // non-zero: the counter-form combine multicasts rows (tokens replicated on all ranks)

  // rank-local state (plain device memory)
  uint32_t* iter;         // dispatch iteration counter; its parity selects the flag set
  uint32_t* comb_iter;    // number of dispatches started = ordinal of the coming combine
  uint32_t* recv_count;   // [nle] rows received per local expert by the last dispatch
  uint2* row_src;         // [nle][cap] {src_rank | k << 16, src_token} per received row
  Status* status;
  uint64_t timeout_ns;
  uint64_t* trace;        // optional [kTraceSlots] %globaltimer stamps of block 0, or null
};

// Trace slots.  0..31: phase stamps of block 0, thread 0 (dispatch 0..15, combine
// 16..31).  Then four arrays of kTraceBlocks stamps taken by thread 0 of every
// block: dispatch start, dispatch end, combine start, combine end.
constexpr int kTraceBlocks = 256;
constexpr int kTraceSlots = 32 + 4 * kTraceBlocks;
constexpr int kTrBlockDispatchStart = 32;
constexpr int kTrBlockDispatchEnd = 32 + kTraceBlocks;
constexpr int kTrBlockCombineStart = 32 + 2 * kTraceBlocks;
constexpr int kTrBlockCombineEnd = 32 + 3 * kTraceBlocks;
enum TraceSlot : int {
  kTrDispatchStart = 0,
  kTrDispatchHist = 1,      // histogram of indices done
  kTrDispatchPosted = 2,    // counts posted, slot bases ready
  kTrDispatchStored = 3,    // this block's payload stores issued
  kTrDispatchSignalled = 4, // arrival counters bumped (end of send)
  kTrDispatchCounts = 5,    // all peers' counts seen
  kTrDispatchLayout = 6,    // row offsets ready
  kTrDispatchCopied = 7,    // this block's rows copied out
  kTrDispatchEnd = 8,
  kTrCombineStart = 16,
  kTrCombineLayout = 17,
  kTrCombineSent = 18,
  kTrCombineReduced = 19,
  kTrCombineEnd = 20,
};

struct DispatchArgs {
  A2AParams p;
  int32_t* out_num_tokens;   // [nle]
  uint8_t* out_x;            // [nle][cap][hidden_bytes]
  int64_t out_x_stride_e;    // bytes
  int64_t out_x_stride_row;  // bytes
  float* out_scale;          // optional, element strides below
  int64_t out_scale_stride_e;
  int64_t out_scale_stride_row;
  int64_t out_scale_stride_col;
  const uint8_t* x;          // [m][hidden_bytes]
  int64_t x_stride_row;      // bytes
  const float* x_scale;      // optional
  int64_t x_scale_stride_row;
  int64_t x_scale_stride_col;
  const uint32_t* indices;   // [m][topk]
  const uint32_t* bound_m;   // optional device scalar
  int num_tokens;            // indices.size(0)
  int quantize;              // x is bf16 [m][hidden_bytes values]; the send converts it to
                             // e4m3 + one fp32 scale per 128 columns on the fly
  int packed;                // send only: two-hop protocol, rows land at their final,
                             // expert-major position in the destination's staging
  int x_on_host;             // x / x_scale live in mapped pinned host memory
  int stage_tokens;          // x_on_host with the flag-in-data send: token rows a block
                             // fetches into shared memory per round (0: read rows in place)
};

struct CombineArgs {
  A2AParams p;
  void* out_tokens;          // [max_tokens][hidden_dim] of U
  int64_t out_stride_row;    // elements
  const float* weights;      // [m][topk]
  int64_t w_stride_row;
  const void* expert_y;      // [nle][cap][hidden_dim] of T
  int64_t y_stride_e;        // elements
  int64_t y_stride_row;      // elements
  const uint32_t* bound_m;
  int num_tokens;
  int ll;                    // this call uses the flag-in-data staging (send and receive halves
                             // of one combine must agree; the GEMM-epilogue send does not use it)
};

// Arguments of several ranks that share one device, passed to a kernel by value (no
// device-side staging, so the launch can be captured in a CUDA graph).
constexpr int kMaxLocalRanks = 8;
struct DispatchMulti {
  DispatchArgs r[kMaxLocalRanks];
};
struct CombineMulti {
  CombineArgs r[kMaxLocalRanks];
};

// Trailer written after payload + scales in every dispatch slot.
struct SlotTrailer {
  uint32_t token;
  uint32_t k;
  uint32_t local_expert;
  uint32_t reserved;
};

__host__ __device__ inline size_t a2a_counts_index(const A2AParams& p, int parity, int src, int le) {
  return (static_cast<size_t>(parity) * p.world + src) * p.nle + le;
}

}  // namespace pplx
