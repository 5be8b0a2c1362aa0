// Combine: every expert output row travels back to the rank(s) that own the
// token, and each token's top-k rows are reduced with the router weights.
//
// Capability parity: intranode_combine.cu:16-187 and internode_combine.cu:11-147
// of the reference (fused / send-only / recv-only; expert_y in f32, f16 or bf16;
// out_tokens in f16 or bf16; results replicated to every rank of the token's DP
// group; fp32 accumulation in k order with one final cast).  What differs:
//
//  * Staging at the token's home rank is indexed by (token, k), where k came
//    with the dispatch trailer, so the reduction reads top-k consecutive rows
//    and never looks at `indices`.
//  * A sender is one warp per received row: batched 16-byte P2P stores, then a
//    single red.release.sys on the token's arrival counter.  No flag handshake
//    precedes the stores (see a2a_params.h for why a rank cannot run ahead).
//  * The reduction is spread over (token, 256-element chunk) warp units so that a
//    single token still uses many warps, and a unit starts as soon as its own
//    token is complete.
//  * A row is split over several warps when there are fewer rows than warps.
//    Arrival is counted in columns: each part adds the columns it carries, so a
//    token is complete at hidden_dim * top-k whatever split the senders chose (and
//    whatever column blocks a GEMM epilogue sends instead).
//  * Signals are issued once per block and round: all warps store their parts,
//    the block synchronises, and one warp executes a single system-scope fence
//    followed by relaxed adds.  (A fence per warp serialises inside an SM and
//    was the largest item of the first version's latency.)
//  * Flag-in-data mode (a.ll, the default): rows travel as 128-byte lines that carry
//    their own flag (core/ll128.cuh).  The send is a plain loop of line stores with
//    no barrier, fence or counter; the reduction is spread over (token, 4-line
//    group) warp units that poll the top-k copies of their own lines and reduce them
//    as soon as those have landed, so a token's first columns are reduced while its
//    last ones are still on the wire.  The per-token counters are advanced locally
//    so that a later combine in counter mode (after the GEMM-epilogue send) still
//    finds them in step.
//  * Block 0 of the send phase clears the counters of the dispatch that just
//    ended and bumps the iteration counter.  The per-token counters used here
//    are never cleared; see a2a_params.h.  Nothing waits on a last block.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../core/device_utils.cuh"
#include "../core/ll128.cuh"
#include "../core/ptx.cuh"
#include "../core/utils.h"
#include "../core/wait.cuh"
#include "a2a_device.cuh"
#include "a2a_kernels.h"
#include "a2a_params.h"

namespace pplx {
namespace {

constexpr int kCombineThreads = 512;
constexpr uint32_t kMaxSplit = 16;

__device__ __forceinline__ int split_factor(uint32_t rows, uint32_t warps, int nvec) {
  if (rows == 0 || rows >= warps) return 1;
  uint32_t s = warps / rows;
  s = 1u << (31 - __clz(s));
  const uint32_t by_size = max(1, nvec >> 5);
  s = min(s, min(kMaxSplit, 1u << (31 - __clz(by_size))));
  return static_cast<int>(s);
}

struct CombineSmem {
  uint32_t* estart;   // [nle + 1]
  uint32_t* sig_tok;  // [nwarps] token whose part a warp stored in the current pass, or kNoSignal
  uint32_t* sig_grp;  // [nwarps] first rank of the token's DP group
  uint8_t* outbuf;    // [nwarps][512] reduced results of one warp unit, before they are stored
};
constexpr int kOutBufBytes = 512;
constexpr uint32_t kNoSignal = 0xffffffffu;

__device__ __forceinline__ CombineSmem carve(uint32_t* s, int nle) {
  CombineSmem m;
  m.estart = s;
  m.sig_tok = m.estart + nle + 1;
  m.sig_grp = m.sig_tok + kCombineThreads / 32;
  const size_t words = static_cast<size_t>(m.sig_grp + kCombineThreads / 32 - s);
  m.outbuf = reinterpret_cast<uint8_t*>(s) + round_up<size_t>(words * sizeof(uint32_t), 16);
  return m;
}

__device__ __forceinline__ void trace(const A2AParams& p, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.trace[slot] = ptx::globaltimer_ns();
}

__device__ __forceinline__ void trace_block(const A2AParams& p, int first_slot) {
  if (p.trace != nullptr && threadIdx.x == 0 && blockIdx.x < kTraceBlocks)
    p.trace[first_slot + blockIdx.x] = ptx::globaltimer_ns();
}

// ---- 8-element vector helpers ------------------------------------------------

template <typename T>
struct Vec8;

template <>
struct Vec8<float> {
  int4 a, b;
  __device__ __forceinline__ void load_cg(const void* p) {
    a = ptx::ld_cg_v4(p);
    b = ptx::ld_cg_v4(static_cast<const uint8_t*>(p) + 16);
  }
  __device__ __forceinline__ void fma_into(float (&acc)[8], float w) const {
    acc[0] = fmaf(w, __int_as_float(a.x), acc[0]);
    acc[1] = fmaf(w, __int_as_float(a.y), acc[1]);
    acc[2] = fmaf(w, __int_as_float(a.z), acc[2]);
    acc[3] = fmaf(w, __int_as_float(a.w), acc[3]);
    acc[4] = fmaf(w, __int_as_float(b.x), acc[4]);
    acc[5] = fmaf(w, __int_as_float(b.y), acc[5]);
    acc[6] = fmaf(w, __int_as_float(b.z), acc[6]);
    acc[7] = fmaf(w, __int_as_float(b.w), acc[7]);
  }
};

__device__ __forceinline__ float2 unpack2(__half2 h) { return __half22float2(h); }
__device__ __forceinline__ float2 unpack2(__nv_bfloat162 h) { return __bfloat1622float2(h); }

template <typename T2>
struct Vec8Half {
  int4 a;
  __device__ __forceinline__ void load_cg(const void* p) { a = ptx::ld_cg_v4(p); }
  __device__ __forceinline__ void fma_into(float (&acc)[8], float w) const {
    const T2* h = reinterpret_cast<const T2*>(&a);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack2(h[j]);
      acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
      acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
    }
  }
};
template <>
struct Vec8<__half> : Vec8Half<__half2> {};
template <>
struct Vec8<__nv_bfloat16> : Vec8Half<__nv_bfloat162> {};

__device__ __forceinline__ int4 pack8(const float (&acc)[8], __half*) {
  int4 r;
  __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
  return r;
}
__device__ __forceinline__ int4 pack8(const float (&acc)[8], __nv_bfloat16*) {
  int4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  return r;
}

// ---- phases --------------------------------------------------------------------

template <typename T, bool kLines>
__device__ __forceinline__ void send_phase(const CombineArgs& a, const CombineSmem& sm) {
  const A2AParams& p = a.p;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;

  if (blockIdx.x == 0) {
    // The dispatch that produced these rows has finished on this rank: clear the
    // flag set it used and move on to the other one.  No peer can write this set
    // again before it has seen counts of this rank's next dispatch.
    const int parity = static_cast<int>(ptx::ld_volatile(p.iter) & 1u);
    uint32_t* counts = reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_counts) +
                       a2a_counts_index(p, parity, 0, 0);
    uint32_t* arrived =
        reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_arrived) + parity * p.world;
    const int P = p.world * p.nle;
    for (int q = tid; q < P; q += blockDim.x) counts[q] = 0;
    if (tid < p.world) arrived[tid] = 0;
    reset_packed_flags(p, parity);
    __syncthreads();
    if (tid == 0) {
      const uint32_t done = *p.iter;
      // Exactly one dispatch must have started since the last combine.
      const uint32_t started = ptx::ld_volatile(p.comb_iter);
      if (started != done + 1u)
        report_failure(p.status, kOutOfOrder, kPhaseCombinePayload, 0, done + 1u, started, p.rank);
      *p.iter = done + 1u;
    }
  }
  for (int le = tid; le < p.nle; le += blockDim.x) sm.estart[le] = p.recv_count[le];
  __syncthreads();
  if (warp == 0) warp_exclusive_scan_smem(sm.estart, p.nle, lane, true);
  __syncthreads();
  trace(p, kTrCombineLayout);
  const uint32_t total_rows = sm.estart[p.nle];

  const int row_bytes = p.hidden_dim * static_cast<int>(sizeof(T));
  const int nvec = row_bytes >> 4;
  const T* y = static_cast<const T*>(a.expert_y);
  const uint32_t gwarp = blockIdx.x * nwarps + warp;
  const uint32_t gwarps = gridDim.x * nwarps;
  const int split = split_factor(total_rows, gwarps, nvec);
  const uint32_t n_units = total_rows * split;

  if constexpr (kLines) {
    const int nlines = ll::lines_for(row_bytes);
    const uint64_t flag = ll::kCombineTag | static_cast<uint64_t>(ptx::ld_volatile(p.comb_iter));
    for (uint32_t unit = gwarp; unit < n_units; unit += gwarps) {
      const uint32_t f = unit / split;
      const int c = static_cast<int>(unit - f * split);
      const int le = find_group(sm.estart, p.nle, f);
      const uint32_t row = f - sm.estart[le];
      const uint2 rs = p.row_src[static_cast<size_t>(le) * p.cap + row];
      const int src_rank = static_cast<int>(rs.x & 0xffffu);
      const uint32_t k = rs.x >> 16;
      const uint32_t token = rs.y;
      if (token >= static_cast<uint32_t>(p.max_tokens) || k >= static_cast<uint32_t>(p.topk) ||
          src_rank >= p.world) {
        if (lane == 0)
          report_failure(p.status, kBadToken, kPhaseCombinePayload, src_rank, p.max_tokens, token,
                         p.rank);
        continue;
      }
      const uint8_t* src = reinterpret_cast<const uint8_t*>(
          y + le * a.y_stride_e + static_cast<int64_t>(row) * a.y_stride_row);
      const int l0 = (c * nlines) / split;
      const int l1 = ((c + 1) * nlines) / split;
      const int group_first = (src_rank / p.dp_size) * p.dp_size;
      for (int r = 0; r < p.dp_size; ++r) {
        uint8_t* slot = p.peer[group_first + r] + p.off_ll_comb_stage +
                        (static_cast<size_t>(token) * p.topk + k) * p.ll_comb_slot_bytes;
        ll::warp_send_lines(slot, src, row_bytes, l0, l1, flag, lane);
      }
    }
    return;
  }

  // With the tokens replicated on all ranks and a multicast mapping of the arena, rows and
  // arrival counts are multicast instead of being sent once per rank.
  const bool to_all = p.mc != nullptr && p.mc_combine != 0;
  // Rounds: in each, every warp stores at most one part; then one fence and the
  // adds for the whole block.  All warps take part in every round's barriers.
  const uint32_t rounds = ceil_div<uint32_t>(n_units, gwarps);
  for (uint32_t round = 0; round < rounds; ++round) {
    const uint32_t unit = round * gwarps + gwarp;
    uint32_t sig_token = kNoSignal;
    uint32_t sig_group = 0;
    uint32_t sig_units = 0;  // columns this warp's part carries
    if (unit < n_units) {
      const uint32_t f = unit / split;
      const int c = static_cast<int>(unit - f * split);
      const int le = find_group(sm.estart, p.nle, f);
      const uint32_t row = f - sm.estart[le];
      const uint2 rs = p.row_src[static_cast<size_t>(le) * p.cap + row];
      const int src_rank = static_cast<int>(rs.x & 0xffffu);
      const uint32_t k = rs.x >> 16;
      const uint32_t token = rs.y;
      if (p.debug_checks && (token >= static_cast<uint32_t>(p.max_tokens) ||
                             k >= static_cast<uint32_t>(p.topk) || src_rank >= p.world)) {
        if (lane == 0)
          report_failure(p.status, kBadToken, kPhaseCombinePayload, src_rank, p.max_tokens,
                         token, p.rank);
      } else {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(
            y + le * a.y_stride_e + static_cast<int64_t>(row) * a.y_stride_row);
        const size_t v0 = static_cast<size_t>((c * nvec) / split);
        const int nv = ((c + 1) * nvec) / split - static_cast<int>(v0);
        const int group_first = (src_rank / p.dp_size) * p.dp_size;
        if (to_all) {
          // Every rank holds the token: the row leaves this GPU once and the NVSwitch
          // delivers it to all of them.
          uint8_t* slot = p.mc + p.off_comb_stage +
                          (static_cast<size_t>(token) * p.topk + k) * row_bytes;
          ptx::warp_copy_v4_multicast<8>(slot + (v0 << 4), src + (v0 << 4), nv, lane);
        } else {
          for (int r = 0; r < p.dp_size; ++r) {
            uint8_t* slot = p.peer[group_first + r] + p.off_comb_stage +
                            (static_cast<size_t>(token) * p.topk + k) * row_bytes;
            // 16 loads in flight per lane: half of a 14 KiB bf16 row in one round trip.
            ptx::warp_copy_v4<ptx::LoadKind::kNonCoherent, 16>(slot + (v0 << 4), src + (v0 << 4),
                                                               nv, lane);
          }
        }
        sig_token = token;
        sig_group = static_cast<uint32_t>(group_first);
        sig_units = static_cast<uint32_t>(nv) * (16u / static_cast<uint32_t>(sizeof(T)));
      }
    }
    if (lane == 0) {
      sm.sig_tok[warp] = sig_token;
      sm.sig_grp[warp] = sig_group | (sig_units << 8);  // ranks fit in 8 bits
    }
    __syncthreads();
    if (warp == 0) {
      const uint32_t tok = lane < nwarps ? sm.sig_tok[lane] : kNoSignal;
      const uint32_t packed_grp = lane < nwarps ? sm.sig_grp[lane] : 0u;
      const uint32_t grp = packed_grp & 0xffu;
      const uint32_t arrival_units = packed_grp >> 8;
      if (__any_sync(0xffffffffu, tok != kNoSignal)) ptx::fence_acq_rel_sys();
      if (tok != kNoSignal && to_all) {
        ptx::multimem_red_add_release_sys(
            reinterpret_cast<uint32_t*>(p.mc + p.off_comb_arrived) + tok, arrival_units);
      } else if (tok != kNoSignal) {
        for (int r = 0; r < p.dp_size; ++r) {
          ptx::red_add_relaxed_sys(
              reinterpret_cast<uint32_t*>(p.peer[grp + r] + p.off_comb_arrived) + tok,
              arrival_units);
        }
      }
    }
    __syncthreads();
  }
}

// 8 bytes of a row of T as floats, accumulated with weight w into acc[0 .. kPer).
template <typename T>
struct Half8;
template <>
struct Half8<float> {
  static constexpr int kPer = 2;
  static __device__ __forceinline__ void fma(float* acc, uint64_t v, float w) {
    acc[0] = fmaf(w, __uint_as_float(static_cast<uint32_t>(v)), acc[0]);
    acc[1] = fmaf(w, __uint_as_float(static_cast<uint32_t>(v >> 32)), acc[1]);
  }
};
template <typename T2>
struct Half8Of16 {
  static constexpr int kPer = 4;
  static __device__ __forceinline__ void fma(float* acc, uint64_t v, float w) {
    const uint32_t lo = static_cast<uint32_t>(v), hi = static_cast<uint32_t>(v >> 32);
    const float2 f0 = unpack2(*reinterpret_cast<const T2*>(&lo));
    const float2 f1 = unpack2(*reinterpret_cast<const T2*>(&hi));
    acc[0] = fmaf(w, f0.x, acc[0]);
    acc[1] = fmaf(w, f0.y, acc[1]);
    acc[2] = fmaf(w, f1.x, acc[2]);
    acc[3] = fmaf(w, f1.y, acc[3]);
  }
};
template <>
struct Half8<__half> : Half8Of16<__half2> {};
template <>
struct Half8<__nv_bfloat16> : Half8Of16<__nv_bfloat162> {};

__device__ __forceinline__ uint32_t pack2(float a, float b, __half*) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16*) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Puts kPer consecutive results (2 or 4), converted to U, at `dst` in shared memory.
template <int kPer, typename U>
__device__ __forceinline__ void stage_results(uint8_t* dst, const float* acc) {
  if constexpr (kPer == 4) {
    uint2 v;
    v.x = pack2(acc[0], acc[1], static_cast<U*>(nullptr));
    v.y = pack2(acc[2], acc[3], static_cast<U*>(nullptr));
    *reinterpret_cast<uint2*>(dst) = v;
  } else {
    *reinterpret_cast<uint32_t*>(dst) = pack2(acc[0], acc[1], static_cast<U*>(nullptr));
  }
}

// Reduction of the flag-in-data mode.  A warp unit is (token, group of four lines): lane
// (g, j) owns the 16 bytes at line 4c + g, offset 16 j of each of the token's top-k rows,
// polls until all of them carry this combine's flag, and reduces them.  The unit's results
// (480 bytes of 16-bit values, 240 for fp32 inputs: a multiple of 16 at a multiple of 16) pass
// through shared memory so that they leave as aligned 16-byte stores, whole lines at a time --
// which matters most when out_tokens is pinned host memory and every store crosses PCIe.
template <typename T, typename U>
__device__ __forceinline__ void recv_phase_ll(const CombineArgs& a, const CombineSmem& sm, int m) {
  const A2AParams& p = a.p;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int j = lane & 7, g = lane >> 3;
  const WaitCtx w{p.status, p.timeout_ns, static_cast<uint32_t>(p.rank)};
  constexpr int kPer = Half8<T>::kPer;

  const int topk = p.topk;
  const int row_bytes = p.hidden_dim * static_cast<int>(sizeof(T));
  const int nlines = ll::lines_for(row_bytes);
  const int groups = ceil_div<int>(nlines, 4);
  const size_t slot_bytes = static_cast<size_t>(p.ll_comb_slot_bytes);
  const uint8_t* stage = p.peer[p.rank] + p.off_ll_comb_stage;
  const uint64_t flag = ll::kCombineTag | static_cast<uint64_t>(ptx::ld_volatile(p.comb_iter));
  U* out = static_cast<U*>(a.out_tokens);

  if (blockIdx.x == 0) {
    // Nobody adds to the per-token counters in this mode; advance them all by one
    // combine's worth so that the counter mode finds them in step afterwards.
    uint32_t* arrived = reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_comb_arrived);
    const uint32_t per_round = static_cast<uint32_t>(topk) * static_cast<uint32_t>(p.comb_units);
    for (int i = tid; i < p.max_tokens; i += blockDim.x) atomicAdd(arrived + i, per_round);
  }

  const uint32_t units = static_cast<uint32_t>(m) * groups;
  const uint32_t gwarp = blockIdx.x * nwarps + warp;
  const uint32_t gwarps = gridDim.x * nwarps;
  for (uint32_t u = gwarp; u < units; u += gwarps) {
    const int i = u / groups;
    const int c = u - i * groups;
    const int line = 4 * c + g;
    const bool live = line < nlines;
    const int o = line * ll::kLineData + j * 16;  // byte offset inside the row of T
    const uint8_t* base = stage + static_cast<size_t>(i) * topk * slot_bytes +
                          static_cast<size_t>(line) * ll::kLineBytes + j * 16;
    const float* wrow = a.weights + static_cast<int64_t>(i) * a.w_stride_row;
    float acc[2 * kPer];
#pragma unroll
    for (int t = 0; t < 2 * kPer; ++t) acc[t] = 0.f;
    ll::Poll poll(w, kPhaseCombinePayload, static_cast<uint32_t>(i));
    bool ok = true;
    constexpr int kBatch = 8;
    for (int k0 = 0; k0 < topk; k0 += kBatch) {
      uint64_t xa[kBatch], xb[kBatch];
      while (true) {
        bool ready = true;
        uint64_t seen = flag;
#pragma unroll
        for (int t = 0; t < kBatch; ++t) {
          if (live && k0 + t < topk) {
            ll::ld16(base + static_cast<size_t>(k0 + t) * slot_bytes, xa[t], xb[t]);
            if (j == 7 && xb[t] != flag) {
              ready = false;
              seen = xb[t];
            }
          }
        }
        if (__all_sync(0xffffffffu, ready)) break;
        if (!poll.again(lane, flag, seen)) {
          ok = false;
          break;
        }
      }
      if (!ok) break;
#pragma unroll
      for (int t = 0; t < kBatch; ++t) {
        if (live && k0 + t < topk) {
          const float wk = __ldg(wrow + k0 + t);
          Half8<T>::fma(acc, xa[t], wk);
          if (j < 7) Half8<T>::fma(acc + kPer, xb[t], wk);
        }
      }
    }
    if (!ok) continue;
    // Bytes of output per byte of input: 1 for 16-bit inputs, 1/2 for fp32.
    constexpr int kIn = static_cast<int>(sizeof(T)), kOut = static_cast<int>(sizeof(U));
    uint8_t* wbuf = sm.outbuf + warp * kOutBufBytes;
    const int in_unit = g * ll::kLineData + j * 16;  // this lane's byte offset inside the unit
    if (live && o + 8 <= row_bytes) stage_results<kPer, U>(wbuf + in_unit / kIn * kOut, acc);
    if (live && j < 7 && o + 16 <= row_bytes)
      stage_results<kPer, U>(wbuf + (in_unit + 8) / kIn * kOut, acc + kPer);
    __syncwarp();
    const int unit_in0 = 4 * c * ll::kLineData;  // first input byte of the unit in its row
    const int out_bytes = (min(row_bytes - unit_in0, 4 * ll::kLineData) / kIn) * kOut;
    uint8_t* out_at = reinterpret_cast<uint8_t*>(out + static_cast<int64_t>(i) * a.out_stride_row) +
                      unit_in0 / kIn * kOut;
    if (lane * 16 < out_bytes)
      ptx::st_v4(out_at + lane * 16, *reinterpret_cast<const int4*>(wbuf + lane * 16));
    __syncwarp();  // the buffer is rewritten by the warp's next unit
  }
  trace(p, kTrCombineReduced);
}

template <typename T, typename U>
__device__ __forceinline__ void recv_phase(const CombineArgs& a, const CombineSmem& sm, int m) {
  const A2AParams& p = a.p;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const WaitCtx w{p.status, p.timeout_ns, static_cast<uint32_t>(p.rank)};

  const int topk = p.topk;
  const int nvec8 = p.hidden_dim >> 3;          // 8-element vectors per row
  const int chunks = ceil_div<int>(nvec8, 32);  // warp units per token
  const int row_bytes = p.hidden_dim * static_cast<int>(sizeof(T));
  const uint8_t* stage = p.peer[p.rank] + p.off_comb_stage;
  uint32_t* arrived = reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_comb_arrived);
  U* out = static_cast<U*>(a.out_tokens);

  const uint32_t units = static_cast<uint32_t>(m) * chunks;
  const uint32_t per_round = static_cast<uint32_t>(topk) * static_cast<uint32_t>(p.comb_units);
  const uint32_t complete = ptx::ld_volatile(p.comb_iter) * per_round;
  if (blockIdx.x == 0) {
    // Tokens beyond bound_m receive nothing in this combine; advance their counters
    // here so that every counter grows by the same amount per combine.
    for (int i = m + tid; i < p.max_tokens; i += blockDim.x) atomicAdd(arrived + i, per_round);
  }
  const uint32_t gwarp = blockIdx.x * nwarps + warp;
  const uint32_t gwarps = gridDim.x * nwarps;
  for (uint32_t u = gwarp; u < units; u += gwarps) {
    const int i = u / chunks;
    const int c = u - i * chunks;
    bool ok = true;
    if (lane == 0) {
      uint32_t seen;
      ok = wait_until(arrived + i, PredReached{complete}, seen, w, kPhaseCombinePayload, i,
                      complete);
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    if (!ok) continue;
    const int v = c * 32 + lane;
    if (v >= nvec8) continue;

    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const uint8_t* base = stage + static_cast<size_t>(i) * topk * row_bytes +
                          static_cast<size_t>(v) * 8 * sizeof(T);
    const float* wrow = a.weights + static_cast<int64_t>(i) * a.w_stride_row;
    constexpr int kBatch = 8;
    for (int k0 = 0; k0 < topk; k0 += kBatch) {
      Vec8<T> x[kBatch];
      float wk[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (k0 + j < topk) {
          x[j].load_cg(base + static_cast<size_t>(k0 + j) * row_bytes);
          wk[j] = __ldg(wrow + k0 + j);
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (k0 + j < topk) x[j].fma_into(acc, wk[j]);
      }
    }
    const int4 packed = pack8(acc, static_cast<U*>(nullptr));
    ptx::st_v4(out + static_cast<int64_t>(i) * a.out_stride_row + static_cast<int64_t>(v) * 8,
               packed);
  }

  trace(p, kTrCombineReduced);
}

// kLines: flag-in-data lines, else counters.  Separate instantiations keep each kernel's code
// small, which counts at decode sizes where the instructions are fetched from DRAM too.
template <typename T, typename U, bool SEND, bool RECV, bool kLines>
__device__ __forceinline__ void combine_body(const CombineArgs& a, uint32_t* smem) {
  const A2AParams& p = a.p;
  const CombineSmem sm = carve(smem, p.nle);
  int m = a.num_tokens;
  if (a.bound_m != nullptr) m = min(m, static_cast<int>(__ldg(a.bound_m)));
  m = min(m, p.max_tokens);
  trace(p, kTrCombineStart);
  trace_block(p, kTrBlockCombineStart);
  if constexpr (SEND) send_phase<T, kLines>(a, sm);
  trace(p, kTrCombineSent);
  if constexpr (SEND && RECV) __syncthreads();
  if constexpr (RECV) {
    if constexpr (kLines) recv_phase_ll<T, U>(a, sm, m);
    else recv_phase<T, U>(a, sm, m);
  }
  trace(p, kTrCombineEnd);
  __syncthreads();
  trace_block(p, kTrBlockCombineEnd);
}

template <typename T, typename U, bool SEND, bool RECV, bool kLines>
__global__ void __launch_bounds__(kCombineThreads, 1)
    combine_kernel(const __grid_constant__ CombineArgs a) {
  extern __shared__ __align__(16) uint32_t dyn_smem[];
  combine_body<T, U, SEND, RECV, kLines>(a, dyn_smem);
}

template <typename T, typename U, bool SEND, bool RECV, bool kLines>
__global__ void __launch_bounds__(kCombineThreads, 1)
    combine_kernel_multi(const __grid_constant__ CombineMulti m) {
  extern __shared__ __align__(16) uint32_t dyn_smem[];
  combine_body<T, U, SEND, RECV, kLines>(m.r[blockIdx.y], dyn_smem);
}

template <typename T, typename U, bool kLines, bool kMulti>
const void* combine_fn(bool send, bool recv) {
  if constexpr (kMulti) {
    if (send && recv) return reinterpret_cast<const void*>(&combine_kernel_multi<T, U, true, true, kLines>);
    if (send) return reinterpret_cast<const void*>(&combine_kernel_multi<T, U, true, false, kLines>);
    return reinterpret_cast<const void*>(&combine_kernel_multi<T, U, false, true, kLines>);
  } else {
    if (send && recv) return reinterpret_cast<const void*>(&combine_kernel<T, U, true, true, kLines>);
    if (send) return reinterpret_cast<const void*>(&combine_kernel<T, U, true, false, kLines>);
    return reinterpret_cast<const void*>(&combine_kernel<T, U, false, true, kLines>);
  }
}

template <typename T, typename U>
cudaError_t launch_typed(const CombineArgs& a, bool send, bool recv, int grid, size_t smem,
                         cudaStream_t stream) {
  const void* fn = a.ll ? combine_fn<T, U, true, false>(send, recv)
                        : combine_fn<T, U, false, false>(send, recv);
  void* params[] = {const_cast<CombineArgs*>(&a)};
  return cudaLaunchKernel(fn, dim3(grid), dim3(kCombineThreads), params, smem, stream);
}

template <typename T, typename U>
cudaError_t launch_typed_multi(const CombineMulti& args, int nranks, bool send, bool recv,
                               int grid, size_t smem, cudaStream_t stream) {
  // All ranks of an emulated world run one instantiation.
  for (int r = 1; r < nranks; ++r) {
    if ((args.r[r].ll != 0) != (args.r[0].ll != 0)) return cudaErrorInvalidValue;
  }
  void* params[] = {const_cast<CombineMulti*>(&args)};
  const void* fn = args.r[0].ll ? combine_fn<T, U, true, true>(send, recv)
                                : combine_fn<T, U, false, true>(send, recv);
  return cudaLaunchCooperativeKernel(fn, dim3(grid, nranks), dim3(kCombineThreads), params, smem,
                                     stream);
}

// Calls fn.template operator()<T, U>() for the (in, out) dtype pair.
template <typename F>
cudaError_t dispatch_types(DType in, DType out, F&& fn) {
  const bool out_bf16 = out == DType::kBF16;
  if (out != DType::kBF16 && out != DType::kF16) return cudaErrorInvalidValue;
  switch (in) {
    case DType::kF32:
      return out_bf16 ? fn.template operator()<float, __nv_bfloat16>()
                      : fn.template operator()<float, __half>();
    case DType::kF16:
      return out_bf16 ? fn.template operator()<__half, __nv_bfloat16>()
                      : fn.template operator()<__half, __half>();
    case DType::kBF16:
      return out_bf16 ? fn.template operator()<__nv_bfloat16, __nv_bfloat16>()
                      : fn.template operator()<__nv_bfloat16, __half>();
  }
  return cudaErrorInvalidValue;
}

}  // namespace

size_t combine_smem_bytes(const A2AParams& p) {
  const size_t words = static_cast<size_t>(p.nle) + 1 + 2 * (kCombineThreads / 32);
  return round_up<size_t>(sizeof(uint32_t) * words, 16) + (kCombineThreads / 32) * kOutBufBytes;
}

int combine_threads() { return kCombineThreads; }

cudaError_t launch_combine(const CombineArgs& a, DType in, DType out, bool send, bool recv,
                           int grid, cudaStream_t stream) {
  const size_t smem = combine_smem_bytes(a.p);
  return dispatch_types(in, out, [&]<typename T, typename U>() {
    return launch_typed<T, U>(a, send, recv, grid, smem, stream);
  });
}

cudaError_t launch_combine_multi(const CombineMulti& args, int nranks, DType in, DType out,
                                 bool send, bool recv, int grid, cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxLocalRanks) return cudaErrorInvalidValue;
  const size_t smem = combine_smem_bytes(args.r[0].p);
  return dispatch_types(in, out, [&]<typename T, typename U>() {
    return launch_typed_multi<T, U>(args, nranks, send, recv, grid, smem, stream);
  });
}

}  // namespace pplx
