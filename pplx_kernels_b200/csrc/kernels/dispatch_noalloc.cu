// Implementation of pplx_b200_dispatch_single_rank_noalloc (see the header for
// the contract).  The kernel is a single-rank variant of the dispatch kernel:
// same two phases (scatter rows into staging sorted by expert, then gather them
// into the caller's per-expert buffers once an arrival counter says the staging
// is complete), but the staging and the counter live in a fixed __device__ array
// instead of an arena that the host allocated.
#include "dispatch_noalloc.h"

#include <cstdio>
#include <mutex>

#include "../core/device_utils.cuh"
#include "../core/ptx.cuh"
#include "../core/utils.h"

namespace {

constexpr size_t kStageBytes = size_t{16} << 20;
constexpr size_t kCtrlBytes = 256;
constexpr int kMaxExperts = 1024;
constexpr int kThreads = 512;
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

// [0, 256): control words (word 0 = rows landed in staging); then the staging rows.
// In host code this name is only a handle for cudaGetSymbolAddress, never a
// device address.
static __device__ __align__(256) uint8_t g_noalloc_scratch[kCtrlBytes + kStageBytes];

struct NoAllocArgs {
  uint8_t* scratch;  // device address of g_noalloc_scratch
  int32_t* out_num_tokens;
  uint8_t* out_x;
  int64_t out_x_stride_e, out_x_stride_row;
  int64_t out_rows;
  float* out_scale;
  int64_t out_scale_stride_e, out_scale_stride_row, out_scale_stride_col;
  const uint8_t* x;
  int64_t x_stride_row;
  const float* x_scale;
  int64_t x_scale_stride_row, x_scale_stride_col;
  const uint32_t* indices;
  const uint32_t* bound_m;
  uint32_t* status;
  int num_tokens, num_experts, topk, hidden_bytes, scale_bytes, slot_bytes;
};

__global__ void __launch_bounds__(kThreads, 1)
    dispatch_single_rank_noalloc_kernel(const __grid_constant__ NoAllocArgs a) {
  using namespace pplx;
  extern __shared__ __align__(16) uint32_t smem[];
  const int E = a.num_experts;
  uint32_t* hist = smem;            // [E]      rows per expert
  uint32_t* base = hist + E;        // [E]      rows of earlier blocks, then running cursor
  uint32_t* estart = base + E;      // [E + 1]  first staging row of each expert
  uint32_t* misc = estart + E + 1;  // [2]      rows stored by this block, wait outcome

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  uint32_t* landed = reinterpret_cast<uint32_t*>(a.scratch);
  uint8_t* stage = a.scratch + kCtrlBytes;

  int m = a.num_tokens;
  if (a.bound_m != nullptr) m = min(m, static_cast<int>(__ldg(a.bound_m)));
  const int per_block = ceil_div<int>(m, gridDim.x);
  const int t_begin = min(static_cast<int>(blockIdx.x) * per_block, m);
  const int t_end = min(t_begin + per_block, m);

  for (int e = tid; e < E; e += blockDim.x) {
    hist[e] = 0;
    base[e] = 0;
  }
  if (tid == 0) {
    misc[0] = 0;
    misc[1] = 1;
  }
  if (blockIdx.x == 0 && tid == 0 && a.status != nullptr) *a.status = 0;
  __syncthreads();
  for (int idx = tid; idx < m * a.topk; idx += blockDim.x) {
    const uint32_t e = __ldg(a.indices + idx);
    if (e < static_cast<uint32_t>(E)) {
      atomicAdd(&hist[e], 1u);
      if (idx / a.topk < t_begin) atomicAdd(&base[e], 1u);
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    estart[e] = hist[e];
    if (blockIdx.x == 0) a.out_num_tokens[e] = static_cast<int32_t>(hist[e]);
  }
  __syncthreads();
  if (warp == 0) warp_exclusive_scan_smem(estart, E, lane, true);
  __syncthreads();
  const uint32_t total_rows = estart[E];

  // Phase 1: rows of this block's tokens -> staging, grouped by expert.
  const int nvec = a.hidden_bytes >> 4;
  const int nscale = a.scale_bytes >> 2;
  for (int u = t_begin * a.topk + warp; u < t_end * a.topk; u += nwarps) {
    const int i = u / a.topk;
    const uint32_t e = __ldg(a.indices + u);
    if (e >= static_cast<uint32_t>(E)) continue;
    uint32_t pos = 0;
    if (lane == 0) {
      pos = estart[e] + atomicAdd(&base[e], 1u);
      atomicAdd(&misc[0], 1u);
    }
    pos = __shfl_sync(0xffffffffu, pos, 0);
    uint8_t* slot = stage + static_cast<size_t>(pos) * a.slot_bytes;
    ptx::warp_copy_v4<ptx::LoadKind::kNonCoherent>(slot, a.x + i * a.x_stride_row, nvec, lane);
    if (nscale > 0) {
      float* sdst = reinterpret_cast<float*>(slot + a.hidden_bytes);
      const float* ssrc = a.x_scale + i * a.x_scale_stride_row;
      for (int j = lane; j < nscale; j += 32) sdst[j] = __ldg(ssrc + j * a.x_scale_stride_col);
    }
  }
  __syncthreads();
  if (tid == 0 && misc[0] > 0) {
    __threadfence();
    atomicAdd(landed, misc[0]);
  }

  // Phase 2: staging -> the caller's per-expert buffers, once every row landed.
  if (tid == 0) {
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::ld_acquire_sys(landed) < total_rows) {
      if (ptx::globaltimer_ns() - t0 > kWaitLimitNs) {
        misc[1] = 0;
        if (a.status != nullptr) *a.status = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (misc[1] == 0) return;
  const uint32_t gwarp = blockIdx.x * nwarps + warp, gwarps = gridDim.x * nwarps;
  for (uint32_t f = gwarp; f < total_rows; f += gwarps) {
    const int e = find_group(estart, E, f);
    const uint32_t row = f - estart[e];
    if (row >= static_cast<uint64_t>(a.out_rows)) continue;
    const uint8_t* slot = stage + static_cast<size_t>(f) * a.slot_bytes;
    ptx::warp_copy_v4<ptx::LoadKind::kL2Only>(
        a.out_x + e * a.out_x_stride_e + static_cast<int64_t>(row) * a.out_x_stride_row, slot, nvec,
        lane);
    if (nscale > 0) {
      const float* ssrc = reinterpret_cast<const float*>(slot + a.hidden_bytes);
      float* sdst = a.out_scale + e * a.out_scale_stride_e +
                    static_cast<int64_t>(row) * a.out_scale_stride_row;
      for (int j = lane; j < nscale; j += 32) sdst[j * a.out_scale_stride_col] = __ldcg(ssrc + j);
    }
  }
}

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
uint8_t* g_scratch_addr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};

int fail(int code, char* msg, size_t len, const char* text) {
  if (msg != nullptr && len > 0) std::snprintf(msg, len, "%s", text);
  return code;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int pplx_b200_dispatch_single_rank_noalloc(
    int32_t* out_expert_num_tokens, void* out_expert_x, int64_t out_x_stride_expert,
    int64_t out_x_stride_row, int64_t out_rows_per_expert, float* out_expert_x_scale,
    int64_t out_scale_stride_expert, int64_t out_scale_stride_row, int64_t out_scale_stride_col,
    const void* x, int64_t x_stride_row, const float* x_scale, int64_t x_scale_stride_row,
    int64_t x_scale_stride_col, const uint32_t* indices, const uint32_t* bound_m, int num_tokens,
    int num_experts, int experts_per_token, int hidden_dim_bytes, int hidden_dim_scale_bytes,
    uint32_t* status, cudaStream_t stream, char* error_message, size_t error_message_len) {
  char* msg = error_message;
  const size_t len = error_message_len;
  if (out_expert_num_tokens == nullptr || out_expert_x == nullptr || x == nullptr ||
      indices == nullptr)
    return fail(kPplxNoAllocBadArgument, msg, len, "a required pointer is null");
  if (num_tokens < 0 || num_experts <= 0 || experts_per_token <= 0 || out_rows_per_expert <= 0)
    return fail(kPplxNoAllocBadArgument, msg, len, "sizes must be positive");
  if (hidden_dim_bytes <= 0 || hidden_dim_bytes % 16 != 0 || hidden_dim_scale_bytes < 0 ||
      hidden_dim_scale_bytes % 4 != 0)
    return fail(kPplxNoAllocBadArgument, msg, len,
                "hidden_dim_bytes must be a positive multiple of 16 and "
                "hidden_dim_scale_bytes a multiple of 4");
  if ((hidden_dim_scale_bytes > 0) != (x_scale != nullptr) ||
      (hidden_dim_scale_bytes > 0) != (out_expert_x_scale != nullptr))
    return fail(kPplxNoAllocBadArgument, msg, len,
                "scale tensors must be given exactly when hidden_dim_scale_bytes > 0");
  if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(out_expert_x) % 16 != 0 ||
      x_stride_row % 16 != 0 || out_x_stride_row % 16 != 0 || out_x_stride_expert % 16 != 0)
    return fail(kPplxNoAllocBadArgument, msg, len, "token buffers must be 16-byte aligned");
  if (num_experts > kMaxExperts)
    return fail(kPplxNoAllocTooLarge, msg, len, "num_experts exceeds the maximum of 1024");
  if (experts_per_token > num_experts)
    return fail(kPplxNoAllocBadArgument, msg, len, "experts_per_token exceeds num_experts");
  const size_t slot_bytes =
      pplx::round_up<size_t>(static_cast<size_t>(hidden_dim_bytes) + hidden_dim_scale_bytes, 16);
  // Checked by division so that no product can wrap: rows that fit into the staging.
  const size_t rows_that_fit = kStageBytes / slot_bytes;
  const size_t need = static_cast<size_t>(num_tokens) * experts_per_token * slot_bytes;
  if (static_cast<size_t>(num_tokens) > rows_that_fit / static_cast<size_t>(experts_per_token)) {
    char text[200];
    std::snprintf(text, sizeof(text),
                  "num_tokens * experts_per_token * slot_bytes = %zu exceeds the built-in staging "
                  "of %zu bytes",
                  need, kStageBytes);
    return fail(kPplxNoAllocTooLarge, msg, len, text);
  }

  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return fail(static_cast<int>(err), msg, len, cudaGetErrorString(err));
  if (device >= kMaxDevices)
    return fail(kPplxNoAllocBadArgument, msg, len, "device ordinal beyond 63");
  {
    // Once per device, with that device current: the symbol's device address.
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (g_scratch_addr[device] == nullptr) {
      void* p = nullptr;
      err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (err != cudaSuccess) return fail(static_cast<int>(err), msg, len, cudaGetErrorString(err));
      int sms = 0;
      err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
      if (err != cudaSuccess) return fail(static_cast<int>(err), msg, len, cudaGetErrorString(err));
      g_sm_count[device] = sms;
      g_scratch_addr[device] = static_cast<uint8_t*>(p);
    }
  }

  NoAllocArgs a{};
  a.scratch = g_scratch_addr[device];
  a.out_num_tokens = out_expert_num_tokens;
  a.out_x = static_cast<uint8_t*>(out_expert_x);
  a.out_x_stride_e = out_x_stride_expert;
  a.out_x_stride_row = out_x_stride_row;
  a.out_rows = out_rows_per_expert;
  a.out_scale = out_expert_x_scale;
  a.out_scale_stride_e = out_scale_stride_expert;
  a.out_scale_stride_row = out_scale_stride_row;
  a.out_scale_stride_col = out_scale_stride_col;
  a.x = static_cast<const uint8_t*>(x);
  a.x_stride_row = x_stride_row;
  a.x_scale = x_scale;
  a.x_scale_stride_row = x_scale_stride_row;
  a.x_scale_stride_col = x_scale_stride_col;
  a.indices = indices;
  a.bound_m = bound_m;
  a.status = status;
  a.num_tokens = num_tokens;
  a.num_experts = num_experts;
  a.topk = experts_per_token;
  a.hidden_bytes = hidden_dim_bytes;
  a.scale_bytes = hidden_dim_scale_bytes;
  a.slot_bytes = static_cast<int>(slot_bytes);

  // The arrival counter is the only word that must start at zero.
  err = cudaMemsetAsync(a.scratch, 0, kCtrlBytes, stream);
  if (err != cudaSuccess) return fail(static_cast<int>(err), msg, len, cudaGetErrorString(err));
  const int rows = num_tokens * experts_per_token;
  int grid = (rows + 3) / 4;
  if (grid < 1) grid = 1;
  if (grid > g_sm_count[device]) grid = g_sm_count[device];
  const size_t smem = sizeof(uint32_t) * (3 * static_cast<size_t>(num_experts) + 1 + 2);
  dispatch_single_rank_noalloc_kernel<<<grid, kThreads, smem, stream>>>(a);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail(static_cast<int>(err), msg, len, cudaGetErrorString(err));
  return kPplxNoAllocOk;
}
