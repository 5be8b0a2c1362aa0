// Launchers of the all-to-all kernels.  Pure CUDA-runtime interface: no torch
// types, so the host classes and the C++ tests can use it directly.
//
// Role parity: the launch halves of AllToAllIntraNode::dispatch / ::combine
// (intranode_dispatch.cu:288-390, intranode_combine.cu:190-266) in the reference.
#pragma once

#include <cuda_runtime.h>

#include "a2a_params.h"

namespace pplx {

enum class DType : int { kF32 = 0, kF16 = 1, kBF16 = 2 };

inline size_t dtype_size(DType t) { return t == DType::kF32 ? 4 : 2; }

// `stage_tokens`: token rows a block fetches into shared memory per round (DispatchArgs).
size_t dispatch_smem_bytes(const A2AParams& p, int stage_tokens = 0);
// Rows per round that fit the staging budget for this geometry (0: rows too long to stage).
int dispatch_stage_tokens(const A2AParams& p);
int dispatch_threads();

// One rank per device (production path).
cudaError_t launch_dispatch(const DispatchArgs& a, bool send, bool recv, int grid,
                            cudaStream_t stream);

// `nranks` (at most kMaxLocalRanks) ranks that share one device, as one cooperative grid
// of (grid, nranks) blocks; the per-rank arguments travel as a kernel parameter.
cudaError_t launch_dispatch_multi(const DispatchMulti& args, int nranks, bool send, bool recv,
                                  int grid, cudaStream_t stream);

// Decode-sized dispatch (dispatch_tiny.cu): objects of a few tokens per rank, lines only.
bool dispatch_tiny_supports(const A2AParams& p);
int dispatch_tiny_grid(const A2AParams& p, int limit);
cudaError_t launch_dispatch_tiny(const DispatchArgs& a, bool send, bool recv, int grid,
                                 cudaStream_t stream);
cudaError_t launch_dispatch_tiny_multi(const DispatchMulti& args, int nranks, bool send, bool recv,
                                       int grid, cudaStream_t stream);

size_t combine_smem_bytes(const A2AParams& p);
int combine_threads();

// in = dtype of expert_y, out = dtype of out_tokens (f16 or bf16).
cudaError_t launch_combine(const CombineArgs& a, DType in, DType out, bool send, bool recv,
                           int grid, cudaStream_t stream);

cudaError_t launch_combine_multi(const CombineMulti& args, int nranks, DType in, DType out,
                                 bool send, bool recv, int grid, cudaStream_t stream);

}  // namespace pplx
