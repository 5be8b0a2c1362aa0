// Device helpers shared by the kernels that take part in the all-to-all protocol.
#pragma once

#include "a2a_params.h"

namespace pplx {

// Clears the packed-mode flag set of `parity` (all threads of one block call it).
__device__ __forceinline__ void reset_packed_flags(const A2AParams& p, int parity) {
  uint32_t* all = reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_counts_all) +
                  static_cast<size_t>(parity) * p.world * p.num_experts;
  for (int i = threadIdx.x; i < p.world * p.num_experts; i += blockDim.x) all[i] = 0;
  uint32_t* arrived_e = reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_arrived_e) +
                        static_cast<size_t>(parity) * p.nle * p.world;
  for (int i = threadIdx.x; i < p.nle * p.world; i += blockDim.x) arrived_e[i] = 0;
}

}  // namespace pplx
