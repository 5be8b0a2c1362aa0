// Single-rank token dispatch for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference library.
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a CUDA
// graph capture of a host framework that forbids allocation while capturing, in
// a real-time serving loop whose device memory is all handed out at start-up, or behind a
// plugin interface that hands the callee tensors and a stream and nothing else.
// The regular path (`AllToAll` + `dispatch`) allocates its staging arena and
// counters with cudaMalloc when the object is created; this function instead
// keeps its staging in a fixed array that is part of the library image, so the
// caller only ever passes inputs and outputs.
//
// What it computes: exactly what `AllToAll.intranode(world_size=1, dp_size=1)`
// followed by `dispatch(...)` computes -- every (token, k) row is routed to
// expert `indices[token, k]`; `out_expert_num_tokens[e]` receives the number of
// rows of expert e and rows `[0, count)` of `out_expert_x[e]` (and of
// `out_expert_x_scale[e]`) receive the payloads, in unspecified order.
//
// Limits (the call fails with kPplxNoAllocTooLarge beyond them):
//   num_tokens * experts_per_token * slot_bytes <= 16 MiB, where
//   slot_bytes = round_up(hidden_dim_bytes + hidden_dim_scale_bytes, 16);
//   num_experts <= 1024.
// The DeepSeek-V3 shape at 128 tokens (1024 rows of 7392 bytes) fits.
// experts_per_token > num_experts is rejected with kPplxNoAllocBadArgument.
//
// Rows beyond `out_rows_per_expert`: an expert that receives more rows than its
// output holds keeps the first `out_rows_per_expert` of them and drops the rest,
// while `out_expert_num_tokens[e]` still reports the full count -- compare the two
// if the output may be too small (out_rows_per_expert >= num_tokens never drops).
//
// Co-residency: the kernel's blocks wait for one another on a counter in the
// array, so the grid is kept within the number of SMs and relies on all of its
// blocks being resident together.  If another stream's work keeps some of them
// off the GPU for longer than the internal limit of two seconds, the call does
// not hang: the waiting blocks give up, `status` reads 1 and the outputs are
// incomplete.
// Every GPU that loads the library holds the 16 MiB (+ 256 B) array until the
// process exits, whether or not this function is ever called.
//
// Set-up: the first call on each device resolves the device address of the
// array (cudaGetSymbolAddress, with that device current) and caches it.  Make
// that first call before any stream capture begins.
//
// Sharing: all calls on one device use the same array, which keeps the previous
// call's contents.  The function clears the one counter that must start at zero
// (stream-ordered, before the kernel).  Two calls that overlap on the GPU -- on
// different streams, or from different threads without ordering -- race on the
// array and produce garbage; order them on one stream or with events.
//
// It calls no cudaMalloc, cudaFree or other allocating routine, and does not
// synchronise.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

extern "C" {

enum PplxNoAllocResult : int {
  kPplxNoAllocOk = 0,
  kPplxNoAllocBadArgument = -1,
  kPplxNoAllocTooLarge = -2,
  // Positive values are cudaError_t codes from the runtime.
};

// Strides of `out_expert_x` and `x` are in bytes, strides of the scale tensors
// in float elements.  `out_expert_x_scale`, `x_scale` (both or neither),
// `bound_m`, `status` and `error_message` may be null.  `status`, when given, is
// a device word that the kernel sets to 0, or to 1 if an internal wait ran out
// (outputs are then incomplete).  `error_message` receives a NUL-terminated
// explanation when the result is not kPplxNoAllocOk.
int pplx_b200_dispatch_single_rank_noalloc(
    int32_t* out_expert_num_tokens, void* out_expert_x, int64_t out_x_stride_expert,
    int64_t out_x_stride_row, int64_t out_rows_per_expert, float* out_expert_x_scale,
    int64_t out_scale_stride_expert, int64_t out_scale_stride_row, int64_t out_scale_stride_col,
    const void* x, int64_t x_stride_row, const float* x_scale, int64_t x_scale_stride_row,
    int64_t x_scale_stride_col, const uint32_t* indices, const uint32_t* bound_m, int num_tokens,
    int num_experts, int experts_per_token, int hidden_dim_bytes, int hidden_dim_scale_bytes,
    uint32_t* status, cudaStream_t stream, char* error_message, size_t error_message_len);

}  // extern "C"
