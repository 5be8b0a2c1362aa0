// Token dispatch: every rank scatters its tokens to the ranks that own the
// tokens' experts, with P2P stores over NVLink, and gathers what it receives
// into the caller's per-expert buffers.
//
// Capability parity: intranode_dispatch.cu:15-284 and internode_dispatch.cu:14-250
// of the reference (fused / send-only / recv-only, fp8 payload with strided fp32
// scales, device-side bound_m, DP-group work split).  The protocol is new:
//
//  SEND  1. Every block histograms `indices` in shared memory, which yields both
//           the per-expert counts and, for the block's own token range, the
//           number of earlier rows per expert.  No global atomics, no grid sync.
//        2. Block 0 posts the counts (value + 1) to every peer straight away, so
//           receivers can lay out their output while payload is in flight.
//        3. One warp per (token, k) copies payload + scales + trailer into the
//           destination's staging region for this source, at a slot that keeps
//           the region sorted by destination-local expert.
//        4. After a block barrier, one thread per destination adds the number of
//           rows the block stored to the destination's arrival counter with a
//           release at system scope.
//  RECV  1. Every block reads all (source, expert) counts (bounded wait) and
//           derives row offsets (sources in rank order, then a warp scan of the
//           group sizes); block 0 writes the per-expert totals.
//        2. One warp per received row waits (bounded) until its source's arrival
//           counter is complete, then copies slot -> out_expert_x / scale and
//           records (source rank, token, k) for combine.
//        3. Nothing is reset here: the combine that follows clears this parity's
//           counters and bumps the iteration counter (dispatch and combine must
//           alternate, as in the reference).
//
// Packed send (a.packed, used by the fused MoE layer): step 2 posts the whole
// histogram to every peer, every block then waits for all peers' histograms and
// places each row at its final position in the destination's staging -- grouped
// by local expert, then by source rank -- and step 4 signals per (destination,
// expert, source) instead of per destination.
//
// Quantising send (a.quantize): the caller's tokens are bf16 and the wire format
// is fp8 e4m3 with one fp32 scale per 128 columns.  The warp that copies a row
// part converts it on the fly -- amax over each 128-column block (8 lanes x 16
// values, reduced with shuffles), scale = max(amax, 1e-4) / 448, value / scale
// rounded to e4m3 -- so no separate quantisation kernel and no fp8 copy of the
// activations in HBM is needed.
//
// Flag-in-data mode (p.ll, the default for the plain dispatch): step 3 writes each
// row as 128-byte lines that carry their own flag (core/ll128.cuh) and step 4 does
// not exist -- the sender never waits for its stores.  The receiver still lays out
// its output from the counts, then polls each expected row line by line and copies
// it out as soon as it is complete, whatever the rest of its source is doing.  The
// packed and the quantising sends keep the counter protocol.
//
// Rows are split over several warps whenever there are fewer rows than warps, so
// that a single token still moves with the whole block's memory parallelism.
//
// Blocks never wait on other blocks of the same rank, and the send phase never
// waits at all, so the kernel needs no cooperative launch.  In fused mode a
// block may sit in a receive wait while a peer still has blocks to schedule, so
// the host keeps the grid within what is resident at once.
#include <algorithm>

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../core/device_utils.cuh"
#include "../core/ll128.cuh"
#include "../core/ptx.cuh"
#include "../core/utils.h"
#include "../core/wait.cuh"
#include "a2a_kernels.h"
#include "a2a_params.h"

namespace pplx {
namespace {

constexpr int kDispatchThreads = 512;
constexpr int kRowCap = 512;           // rows per block whose slots are precomputed
constexpr uint32_t kNoSlot = 0xffffffffu;

// The wire protocol and payload treatment of a launch.  Each is its own kernel instantiation:
// a decode-sized launch after an L2 flush also fetches its instructions from DRAM, and a
// kernel that carries every variant pays for all of them (3 µs at one token).
enum Mode : int {
  kModeLines = 0,        // flag-in-data lines, rows read where they are
  kModeLinesStaged = 1,  // ... rows fetched from host memory into shared memory first
  kModeCounters = 2,     // stores, barrier, arrival counters
  kModeQuant = 3,        // counters; bf16 -> e4m3 + scales inside the send
  kModePacked = 4,       // counters; two-hop expert-major placement (fused MoE layer)
  kModePackedQuant = 5,  // ... with the quantisation
};
template <int kMode>
struct ModeOf {
  static constexpr bool ll = kMode == kModeLines || kMode == kModeLinesStaged;
  static constexpr bool staged = kMode == kModeLinesStaged;
  static constexpr bool quantize = kMode == kModeQuant || kMode == kModePackedQuant;
  static constexpr bool packed = kMode == kModePacked || kMode == kModePackedQuant;
};

// Number of warps that share one row: the largest power of two that keeps every
// warp busy, at most 16, and never so many that a warp gets under 32 vectors.
__device__ __forceinline__ int split_factor(uint32_t rows, uint32_t warps, int nvec) {
  if (rows == 0 || rows >= warps) return 1;
  uint32_t s = warps / rows;
  s = 1u << (31 - __clz(s));
  const uint32_t by_size = max(1, nvec >> 5);
  s = min(s, min(16u, 1u << (31 - __clz(by_size))));
  return static_cast<int>(s);
}

struct DispatchSmem {
  uint32_t* hist;    // [E]
  uint32_t* base;    // [E]
  uint32_t* off;     // [E]  rows for lower local experts of the same destination
  uint32_t* bef;     // [E]  packed mode: rows that lower-ranked sources send to the expert
  uint32_t* fstart;  // [P + 1]  counts, then their exclusive scan
  uint32_t* rbase;   // [P]
  uint32_t* sent;    // [kMaxWorld]
  uint32_t* rowpos;  // [kRowCap] staging slot of each row this block sends
  uint8_t* xstage;   // token rows fetched from host memory before they are sent (optional)
};

__device__ __forceinline__ DispatchSmem carve(uint32_t* s, int E, int P) {
  DispatchSmem m;
  m.hist = s;
  m.base = m.hist + E;
  m.off = m.base + E;
  m.bef = m.off + E;
  m.fstart = m.bef + E;
  m.rbase = m.fstart + P + 1;
  m.sent = m.rbase + P;
  m.rowpos = m.sent + kMaxWorld;
  // The word arrays before it have an odd total in general; rows are moved with 16-byte
  // accesses, so the staging starts on the next 16-byte boundary of the (16-byte aligned)
  // dynamic shared memory.
  const size_t words = static_cast<size_t>(m.rowpos + kRowCap - s);
  m.xstage = reinterpret_cast<uint8_t*>(s) + round_up<size_t>(words * sizeof(uint32_t), 16);
  return m;
}

__device__ __forceinline__ void trace(const A2AParams& p, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.trace[slot] = ptx::globaltimer_ns();
}

__device__ __forceinline__ void trace_block(const A2AParams& p, int first_slot) {
  if (p.trace != nullptr && threadIdx.x == 0 && blockIdx.x < kTraceBlocks)
    p.trace[first_slot + blockIdx.x] = ptx::globaltimer_ns();
}

__device__ __forceinline__ uint32_t* counts_ptr(const A2AParams& p, int dst, int parity, int src,
                                                int le) {
  return reinterpret_cast<uint32_t*>(p.peer[dst] + p.off_counts) +
         a2a_counts_index(p, parity, src, le);
}

__device__ __forceinline__ uint32_t* arrived_ptr(const A2AParams& p, int dst, int parity, int src) {
  return reinterpret_cast<uint32_t*>(p.peer[dst] + p.off_arrived) + parity * p.world + src;
}

// Quantises columns [16 * v0, 16 * v1) of one bf16 row to e4m3 (v = 16-value output
// vectors; v0 is a multiple of 8 so that 128-column blocks are not split between
// warps) and stores payload and scales into the slot.
__device__ __forceinline__ void warp_quantize_row(uint8_t* slot, float* slot_scales,
                                                  const __nv_bfloat16* src, int v0, int v1,
                                                  int nvec, int lane, bool pow2) {
  for (int base = v0; base < v1; base += 32) {
    const int v = base + lane;
    const bool live = v < v1 && v < nvec;
    float f[16];
    float amax = 0.f;
    if (live) {
      const int4 lo = ptx::ld_nc_v4(src + static_cast<size_t>(v) * 16);
      const int4 hi = ptx::ld_nc_v4(src + static_cast<size_t>(v) * 16 + 8);
      const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&lo);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&hi);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(a[j]);
        const float2 y = __bfloat1622float2(b[j]);
        f[2 * j] = x.x;
        f[2 * j + 1] = x.y;
        f[8 + 2 * j] = y.x;
        f[8 + 2 * j + 1] = y.y;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(f[j]));
    }
    // 8 consecutive lanes hold one 128-column block.
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    if (!live) continue;
    amax = fmaxf(amax, 1e-4f);
    float scale = amax / 448.0f, inv = 448.0f / amax;
    if (pow2) {
      // The smallest power of two that is not below amax / 448: hardware block scaling.
      const uint32_t bits = __float_as_uint(scale);
      scale = __uint_as_float(((bits >> 23) + ((bits & 0x7fffffu) != 0u ? 1u : 0u)) << 23);
      inv = 1.0f / scale;
    }
    uint32_t q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * j] * inv, f[4 * j + 1] * inv),
                                                   __NV_SATFINITE, __NV_E4M3);
      const uint32_t p1 = __nv_cvt_float2_to_fp8x2(
          make_float2(f[4 * j + 2] * inv, f[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
      q[j] = p0 | (p1 << 16);
    }
    int4 out;
    out.x = q[0];
    out.y = q[1];
    out.z = q[2];
    out.w = q[3];
    ptx::st_v4(slot + static_cast<size_t>(v) * 16, out);
    if ((lane & 7) == 0) slot_scales[v >> 3] = scale;
  }
}

template <int kMode>
__device__ __forceinline__ void send_phase(const DispatchArgs& a, const DispatchSmem& sm,
                                           int parity, int m, uint32_t iter_now) {
  using M = ModeOf<kMode>;
  const A2AParams& p = a.p;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int E = p.num_experts;
  const int topk = p.topk;
  const int dp_rank = p.rank % p.dp_size;

  // Rows this rank sends: entry u = o * topk + k of token i = o * dp_size + dp_rank.
  // Blocks own contiguous ranges of u.
  const int n_own = (m > dp_rank) ? (m - dp_rank + p.dp_size - 1) / p.dp_size : 0;
  const int n_entries = n_own * topk;
  const int per_block = ceil_div<int>(n_entries, gridDim.x);
  const int u_begin = min(static_cast<int>(blockIdx.x) * per_block, n_entries);
  const int u_end = min(u_begin + per_block, n_entries);

  // The rows this block will copy are known before their destinations are: ask
  // for them now, so that they arrive in L2 while the histogram is built.
  {
    const int rows_here = u_end - u_begin;
    const int src_bytes = M::quantize ? 2 * p.hidden_bytes : p.hidden_bytes;
    if (rows_here > 0 && rows_here <= kRowCap && !a.x_on_host) {
      const int parts = split_factor(rows_here, nwarps, p.hidden_bytes >> 4);
      for (int unit = warp; unit < rows_here * parts; unit += nwarps) {
        const int r = unit / parts;
        const int c = unit - r * parts;
        const int i = ((u_begin + r) / topk) * p.dp_size + dp_rank;
        const uint8_t* src = a.x + static_cast<int64_t>(i) * a.x_stride_row;
        const int b0 = ((c * src_bytes) / parts) & ~127;
        const int b1 = ((c + 1) * src_bytes) / parts;
        for (int b = b0 + lane * 128; b < b1; b += 32 * 128) ptx::prefetch_l2(src + b);
      }
    }
  }

  for (int e = tid; e < E; e += blockDim.x) {
    sm.hist[e] = 0;
    sm.base[e] = 0;
  }
  if (tid < kMaxWorld) sm.sent[tid] = 0;
  // A new round begins: the combine that follows this dispatch is one further.
  if (blockIdx.x == 0 && tid == 0) {
    const uint32_t started = *p.comb_iter;
    // Dispatches started must equal combines finished: anything else is two dispatches
    // without a combine in between, which the flag protocol does not survive.
    if (started != iter_now)
      report_failure(p.status, kOutOfOrder, kPhaseDispatchCounts, 0, iter_now, started, p.rank);
    *p.comb_iter = started + 1u;
  }
  __syncthreads();

  for (int idx = tid; idx < n_entries; idx += blockDim.x) {
    const int o = idx / topk;
    const int k = idx - o * topk;
    const int i = o * p.dp_size + dp_rank;
    const uint32_t e = __ldg(a.indices + static_cast<size_t>(i) * topk + k);
    if (e < static_cast<uint32_t>(E)) {
      atomicAdd(&sm.hist[e], 1u);
      if (idx < u_begin) atomicAdd(&sm.base[e], 1u);
      // An index in the padding above the configured expert count is delivered to a
      // surplus slot of the last rank; with checks on it is reported as well.
      if (p.debug_checks && e >= static_cast<uint32_t>(p.num_real_experts) && blockIdx.x == 0)
        report_failure(p.status, kBadExpert, kPhaseDispatchCounts, i, p.num_real_experts, e, p.rank);
    } else if (p.debug_checks) {
      report_failure(p.status, kBadExpert, kPhaseDispatchCounts, i, E, e, p.rank);
    }
  }
  __syncthreads();
  trace(p, kTrDispatchHist);

  constexpr bool packed = M::packed;
  constexpr bool ll = M::ll;
  const uint64_t flag = ll::kDispatchTag | static_cast<uint64_t>(iter_now + 1u);
  if (!packed) {
    if (blockIdx.x == 0) {
      for (int e = tid; e < E; e += blockDim.x) {
        const int dst = e / p.nle;
        const int le = e - dst * p.nle;
        ptx::st_relaxed_sys(counts_ptr(p, dst, parity, p.rank, le), sm.hist[e] + 1u);
      }
    }
    for (int e = tid; e < E; e += blockDim.x) sm.off[e] = sm.hist[e];
  } else {
    // Hop 1: everybody learns everybody's histogram.
    const int WE = p.world * E;
    if (blockIdx.x == 0 && p.mc != nullptr) {
      // The same words go to the same place on every rank: one multicast store each, and
      // the NVSwitch replicates them.
      uint32_t* dstp = reinterpret_cast<uint32_t*>(p.mc + p.off_counts_all) +
                       (static_cast<size_t>(parity) * p.world + p.rank) * E;
      for (int e = tid; e < E; e += blockDim.x) ptx::multimem_st_relaxed_sys(dstp + e, sm.hist[e] + 1u);
    } else if (blockIdx.x == 0) {
      for (int idx = tid; idx < WE; idx += blockDim.x) {
        const int d = idx / E;
        const int e = idx - d * E;
        uint32_t* dstp = reinterpret_cast<uint32_t*>(p.peer[d] + p.off_counts_all) +
                         (static_cast<size_t>(parity) * p.world + p.rank) * E + e;
        ptx::st_relaxed_sys(dstp, sm.hist[e] + 1u);
      }
    }
    for (int e = tid; e < E; e += blockDim.x) {
      sm.off[e] = 0;
      sm.bef[e] = 0;
    }
    __syncthreads();
    const WaitCtx w{p.status, p.timeout_ns, static_cast<uint32_t>(p.rank)};
    const uint32_t* all = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.off_counts_all) +
                          static_cast<size_t>(parity) * p.world * E;
    for (int idx = tid; idx < WE; idx += blockDim.x) {
      const int src = idx / E;
      const int e = idx - src * E;
      uint32_t v = 0;
      if (wait_until(all + idx, PredNonZero{}, v, w, kPhaseDispatchCounts, src, 1u) && v > 1u) {
        atomicAdd(&sm.off[e], v - 1u);
        if (src < p.rank) atomicAdd(&sm.bef[e], v - 1u);
      }
    }
  }

  // Slot of the first row this block stores for expert e: rows for lower local
  // experts of the same destination come first (all sources' rows in packed
  // mode), then lower-ranked sources' rows for the expert (packed mode), then
  // earlier blocks' rows.  One warp per destination scans that destination.
  __syncthreads();
  for (int dst = warp; dst < p.world; dst += nwarps) {
    warp_exclusive_scan_smem(sm.off + dst * p.nle, p.nle, lane, false);
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    sm.base[e] += sm.off[e] + (packed ? sm.bef[e] : 0u);
    sm.hist[e] = 0;  // from here on: rows this block stored for expert e (packed mode)
  }
  __syncthreads();

  const int nvec = p.hidden_bytes >> 4;
  const int nscale = p.scale_bytes >> 2;
  const int rows_here = u_end - u_begin;
  const uint32_t slot_limit =
      static_cast<uint32_t>(packed ? p.world * p.region_slots : p.region_slots);
  const size_t region_first = packed ? 0 : static_cast<size_t>(p.rank) * p.region_slots;
  const bool precomputed = rows_here <= kRowCap;
  int split = 1;
  if (precomputed) {
    // Reserve every row's slot up front so that several warps can share a row.
    for (int r = tid; r < rows_here; r += blockDim.x) {
      const int u = u_begin + r;
      const int o = u / topk;
      const int i = o * p.dp_size + dp_rank;
      const uint32_t e = __ldg(a.indices + static_cast<size_t>(i) * topk + (u - o * topk));
      uint32_t pos = kNoSlot;
      if (e < static_cast<uint32_t>(E)) {
        pos = atomicAdd(&sm.base[e], 1u);
        // Always checked: a token that names one expert twice would otherwise push its
        // rows past the region that the distinct-expert rule sizes.
        if (pos >= slot_limit) {
          report_failure(p.status, kSlotOverflow, kPhaseDispatchPayload, e / p.nle, slot_limit,
                         pos, p.rank);
          pos = kNoSlot;
        } else {
          atomicAdd(&sm.sent[e / p.nle], 1u);
          if (packed) atomicAdd(&sm.hist[e], 1u);
        }
      }
      sm.rowpos[r] = pos;
    }
    __syncthreads();
    split = split_factor(rows_here, nwarps, nvec);
  }
  trace(p, kTrDispatchPosted);

  // Tokens whose rows this block sends, taken in chunks.  With the tokens in host memory a
  // chunk is first fetched into shared memory (every byte crosses PCIe once, however many
  // experts the token goes to) and sent from there; otherwise there is one chunk and the
  // rows are read where they are.
  const int stage_tokens = M::staged ? max(a.stage_tokens, 1) : 0;
  const int row_smem = round_up<int>(p.hidden_bytes + p.scale_bytes, 16);
  const int o_first = u_begin / topk;
  const int o_end = rows_here > 0 ? (u_end - 1) / topk + 1 : o_first;
  const int o_step = stage_tokens > 0 ? stage_tokens : max(1, o_end - o_first);
  for (int o0 = o_first; o0 < o_end; o0 += o_step) {
    const int o1 = min(o0 + o_step, o_end);
    if constexpr (M::staged) {
      const int per_row = nvec + nscale;  // 16-byte vectors of payload, then single scales
      for (int idx = tid; idx < (o1 - o0) * per_row; idx += blockDim.x) {
        const int t = idx / per_row;
        const int v = idx - t * per_row;
        const int i = (o0 + t) * p.dp_size + dp_rank;
        uint8_t* row = sm.xstage + static_cast<size_t>(t) * row_smem;
        if (v < nvec) {
          *reinterpret_cast<int4*>(row + (static_cast<size_t>(v) << 4)) =
              ptx::ld_nc_v4(a.x + static_cast<int64_t>(i) * a.x_stride_row + (static_cast<size_t>(v) << 4));
        } else {
          const int j = v - nvec;
          reinterpret_cast<float*>(row + p.hidden_bytes)[j] =
              __ldg(a.x_scale + static_cast<int64_t>(i) * a.x_scale_stride_row +
                    static_cast<int64_t>(j) * a.x_scale_stride_col);
        }
      }
      __syncthreads();
    }
    const int ua = max(u_begin, o0 * topk);
    const int ub = min(u_end, o1 * topk);
    const int n_units = (ub - ua) * split;
    for (int unit = warp; unit < n_units; unit += nwarps) {
      const int r = (ua - u_begin) + unit / split;
      const int c = unit % split;
      const int u = u_begin + r;
      const int o = u / topk;
      const int k = u - o * topk;
      const int i = o * p.dp_size + dp_rank;
      const uint32_t e = __ldg(a.indices + static_cast<size_t>(i) * topk + k);
      if (e >= static_cast<uint32_t>(E)) continue;
      const int dst = e / p.nle;
      const int le = e - dst * p.nle;
      uint32_t pos;
      if (precomputed) {
        pos = sm.rowpos[r];
        if (pos == kNoSlot) continue;
      } else {
        pos = 0;
        if (lane == 0) pos = atomicAdd(&sm.base[e], 1u);
        pos = __shfl_sync(0xffffffffu, pos, 0);
        if (pos >= slot_limit) {
          if (lane == 0)
            report_failure(p.status, kSlotOverflow, kPhaseDispatchPayload, dst, slot_limit, pos,
                           p.rank);
          continue;
        }
        if (lane == 0) {
          atomicAdd(&sm.sent[dst], 1u);
          if (packed) atomicAdd(&sm.hist[e], 1u);
        }
      }

      const uint8_t* src = a.x + static_cast<int64_t>(i) * a.x_stride_row;
      if (ll) {
        uint8_t* slot =
            p.peer[dst] + p.off_ll_disp_stage + (region_first + pos) * p.ll_slot_bytes;
        const int l0 = (c * p.ll_x_lines) / split;
        const int l1 = ((c + 1) * p.ll_x_lines) / split;
        const uint32_t trailer[4] = {static_cast<uint32_t>(i), static_cast<uint32_t>(k),
                                     static_cast<uint32_t>(le), static_cast<uint32_t>(p.rank)};
        uint8_t* meta = slot + p.ll_x_lines * ll::kLineBytes;
        if constexpr (M::staged) {
          const uint8_t* row = sm.xstage + static_cast<size_t>(o - o0) * row_smem;
          ll::warp_send_lines<ll::Src::kShared>(slot, row, p.hidden_bytes, l0, l1, flag, lane);
          if (c == split - 1)
            ll::warp_send_meta<ll::Src::kShared>(
                meta, p.ll_meta_lines, trailer, reinterpret_cast<const float*>(row + p.hidden_bytes),
                1, nscale, flag, lane);
        } else {
          ll::warp_send_lines(slot, src, p.hidden_bytes, l0, l1, flag, lane);
          if (c == split - 1) {
            const float* ssrc =
                nscale > 0 ? a.x_scale + static_cast<int64_t>(i) * a.x_scale_stride_row : nullptr;
            ll::warp_send_meta(meta, p.ll_meta_lines, trailer, ssrc, a.x_scale_stride_col, nscale,
                               flag, lane);
          }
        }
        continue;
      }
      uint8_t* slot = p.peer[dst] + p.off_disp_stage + (region_first + pos) * p.slot_bytes;
      if constexpr (M::quantize) {
        // Parts are cut at multiples of 32 output vectors (512 columns).
        const int groups = ceil_div<int>(nvec, 32);
        const int v0 = ((c * groups) / split) * 32;
        const int v1 = min((((c + 1) * groups) / split) * 32, nvec);
        warp_quantize_row(slot, reinterpret_cast<float*>(slot + p.hidden_bytes),
                          reinterpret_cast<const __nv_bfloat16*>(src), v0, v1, nvec, lane,
                          p.quant_pow2 != 0);
      } else {
        const int v0 = (c * nvec) / split;
        const int v1 = ((c + 1) * nvec) / split;
        ptx::warp_copy_v4<ptx::LoadKind::kNonCoherent>(slot + (static_cast<size_t>(v0) << 4),
                                                       src + (static_cast<size_t>(v0) << 4),
                                                       v1 - v0, lane);
      }
      if (c == split - 1) {
        if (nscale > 0 && !M::quantize) {
          float* sdst = reinterpret_cast<float*>(slot + p.hidden_bytes);
          const float* ssrc = a.x_scale + static_cast<int64_t>(i) * a.x_scale_stride_row;
          for (int j = lane; j < nscale; j += 32) sdst[j] = __ldg(ssrc + j * a.x_scale_stride_col);
        }
        if (lane == 0) {
          int4 t;
          t.x = i;
          t.y = k;
          t.z = le;
          t.w = p.rank;
          ptx::st_v4(slot + p.trailer_off, t);
        }
      }
    }
    if constexpr (M::staged) __syncthreads();  // the next chunk overwrites the staged rows
  }
  trace(p, kTrDispatchStored);
  // (Also in flag-in-data mode, where nothing is signalled: warps that ran ahead into the
  // receive phase would poll for counts next to warps that are still storing, and measurably
  // slow them down.)
  __syncthreads();
  if (ll) {
    // Nothing to signal: every line carries its own flag.
  } else if (!packed) {
    if (tid < p.world && sm.sent[tid] > 0) {
      ptx::red_add_release_sys(arrived_ptr(p, tid, parity, p.rank), sm.sent[tid]);
    }
  } else if (warp == 0) {
    // One fence for the block, then one relaxed add per expert that got rows.
    bool any = false;
    for (int d = lane; d < p.world; d += 32) any |= sm.sent[d] > 0;
    if (__any_sync(0xffffffffu, any)) {
      ptx::fence_acq_rel_sys();
      for (int e = lane; e < E; e += 32) {
        const uint32_t n = sm.hist[e];
        if (n == 0) continue;
        const int dst = e / p.nle;
        const int le = e - dst * p.nle;
        ptx::red_add_relaxed_sys(reinterpret_cast<uint32_t*>(p.peer[dst] + p.off_arrived_e) +
                                     (static_cast<size_t>(parity) * p.nle + le) * p.world + p.rank,
                                 n);
      }
    }
  }
  trace(p, kTrDispatchSignalled);
}

template <int kMode>
__device__ __forceinline__ void recv_phase(const DispatchArgs& a, const DispatchSmem& sm,
                                           int parity, uint32_t iter_now) {
  const A2AParams& p = a.p;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int P = p.world * p.nle;
  const WaitCtx w{p.status, p.timeout_ns, static_cast<uint32_t>(p.rank)};
  constexpr bool ll = ModeOf<kMode>::ll;
  const uint64_t flag = ll::kDispatchTag | static_cast<uint64_t>(iter_now + 1u);

  uint32_t* counts = reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_counts) +
                     a2a_counts_index(p, parity, 0, 0);
  uint32_t* arrived =
      reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_arrived) + parity * p.world;

  for (int q = tid; q < P; q += blockDim.x) {
    uint32_t v = 0;
    const bool ok =
        wait_until(counts + q, PredNonZero{}, v, w, kPhaseDispatchCounts, q / p.nle, 1u);
    sm.fstart[q] = ok ? v - 1u : 0u;
  }
  __syncthreads();
  trace(p, kTrDispatchCounts);
  // Row offset of (source s, expert le) inside the expert's output: sources in
  // rank order.
  for (int q = tid; q < P; q += blockDim.x) {
    const int s = q / p.nle;
    const int le = q - s * p.nle;
    uint32_t before = 0;
    for (int s2 = 0; s2 < s; ++s2) before += sm.fstart[s2 * p.nle + le];
    sm.rbase[q] = before;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int le = tid; le < p.nle; le += blockDim.x) {
      const int q = (p.world - 1) * p.nle + le;
      const uint32_t total = sm.rbase[q] + sm.fstart[q];
      a.out_num_tokens[le] = static_cast<int32_t>(total);
      p.recv_count[le] = min(total, static_cast<uint32_t>(p.cap));
    }
  }
  __syncthreads();
  if (warp == 0) warp_exclusive_scan_smem(sm.fstart, P, lane, true);  // first flat row of group q
  __syncthreads();
  trace(p, kTrDispatchLayout);

  const uint32_t total_rows = sm.fstart[P];
  const int nvec = p.hidden_bytes >> 4;
  const int nscale = p.scale_bytes >> 2;
  const uint8_t* stage = p.peer[p.rank] + p.off_disp_stage;
  const uint32_t gwarp = blockIdx.x * nwarps + warp;
  const uint32_t gwarps = gridDim.x * nwarps;

  const int split = split_factor(total_rows, gwarps, nvec);
  const uint32_t n_units = total_rows * split;
  uint32_t acquired = 0;  // sources whose arrival counter this warp has acquired
  for (uint32_t unit = gwarp; unit < n_units; unit += gwarps) {
    const uint32_t f = unit / split;
    const int c = static_cast<int>(unit - f * split);
    const int q = find_group(sm.fstart, P, f);
    const int s = q / p.nle;
    const int le = q - s * p.nle;
    const uint32_t src_first = sm.fstart[s * p.nle];
    const uint32_t src_total = sm.fstart[(s + 1) * p.nle] - src_first;
    const uint32_t slot_idx = f - src_first;
    const uint32_t row = sm.rbase[q] + (f - sm.fstart[q]);

    // Always checked (one compare per row): counts that exceed what the buffers hold.
    if (row >= static_cast<uint32_t>(p.cap) || slot_idx >= static_cast<uint32_t>(p.region_slots)) {
      if (lane == 0)
        report_failure(p.status, kRowOverflow, kPhaseDispatchPayload, s, p.cap, row, p.rank);
      continue;
    }

    if (ll) {
      // Poll the row's own lines; no counter, no acquire: a line is valid as a whole
      // once its flag matches.
      const uint8_t* slot = p.peer[p.rank] + p.off_ll_disp_stage +
                            (static_cast<size_t>(s) * p.region_slots + slot_idx) * p.ll_slot_bytes;
      uint8_t* dst =
          a.out_x + le * a.out_x_stride_e + static_cast<int64_t>(row) * a.out_x_stride_row;
      ll::Poll poll(w, kPhaseDispatchPayload, static_cast<uint32_t>(s));
      const int l0 = (c * p.ll_x_lines) / split;
      const int l1 = ((c + 1) * p.ll_x_lines) / split;
      if (!ll::warp_recv_lines(dst, slot, p.hidden_bytes, l0, l1, flag, lane, poll)) continue;
      if (c == split - 1) {
        uint32_t trailer[4];
        float* sdst = nscale > 0 ? a.out_scale + le * a.out_scale_stride_e +
                                       static_cast<int64_t>(row) * a.out_scale_stride_row
                                 : nullptr;
        if (!ll::warp_recv_meta(slot + p.ll_x_lines * ll::kLineBytes, p.ll_meta_lines, sdst,
                                a.out_scale_stride_col, nscale, flag, lane, poll, trailer))
          continue;
        if (lane == 0) {
          if (trailer[0] >= static_cast<uint32_t>(p.max_tokens) ||
              trailer[1] >= static_cast<uint32_t>(p.topk)) {
            report_failure(p.status, kBadToken, kPhaseDispatchPayload, s, p.max_tokens, trailer[0],
                           p.rank);
          } else {
            uint2 rs;
            rs.x = static_cast<uint32_t>(s) | (trailer[1] << 16);
            rs.y = trailer[0];
            p.row_src[static_cast<size_t>(le) * p.cap + row] = rs;
          }
        }
      }
      continue;
    }

    // Each warp acquires a source's counter itself once; a flag set by another
    // warp would not order this warp's loads after the peer's stores.
    bool ok = true;
    if (!((acquired >> s) & 1u)) {
      if (lane == 0) {
        uint32_t seen;
        ok = wait_until(arrived + s, PredGe{src_total}, seen, w, kPhaseDispatchPayload, s,
                        src_total);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      __syncwarp();
      if (!ok) continue;
      acquired |= 1u << s;
    }
    const uint8_t* slot =
        stage + (static_cast<size_t>(s) * p.region_slots + slot_idx) * p.slot_bytes;
    uint8_t* dst = a.out_x + le * a.out_x_stride_e + static_cast<int64_t>(row) * a.out_x_stride_row;
    const int v0 = (c * nvec) / split;
    const int v1 = ((c + 1) * nvec) / split;
    ptx::warp_copy_v4<ptx::LoadKind::kL2Only>(dst + (static_cast<size_t>(v0) << 4),
                                              slot + (static_cast<size_t>(v0) << 4), v1 - v0, lane);
    if (c == split - 1) {
      if (nscale > 0) {
        const float* ssrc = reinterpret_cast<const float*>(slot + p.hidden_bytes);
        float* sdst = a.out_scale + le * a.out_scale_stride_e +
                      static_cast<int64_t>(row) * a.out_scale_stride_row;
        for (int j = lane; j < nscale; j += 32) sdst[j * a.out_scale_stride_col] = __ldcg(ssrc + j);
      }
      if (lane == 0) {
        const int4 t = ptx::ld_cg_v4(slot + p.trailer_off);
        if (p.debug_checks && static_cast<uint32_t>(t.x) >= static_cast<uint32_t>(p.max_tokens)) {
          report_failure(p.status, kBadToken, kPhaseDispatchPayload, s, p.max_tokens, t.x, p.rank);
        }
        uint2 rs;
        rs.x = static_cast<uint32_t>(s) | (static_cast<uint32_t>(t.y) << 16);
        rs.y = static_cast<uint32_t>(t.x);
        p.row_src[static_cast<size_t>(le) * p.cap + row] = rs;
      }
    }
  }
  trace(p, kTrDispatchCopied);
  trace(p, kTrDispatchEnd);
}

template <bool SEND, bool RECV, int kMode>
__device__ __forceinline__ void dispatch_body(const DispatchArgs& a, uint32_t* smem) {
  const A2AParams& p = a.p;
  const DispatchSmem sm = carve(smem, p.num_experts, p.world * p.nle);
  const uint32_t iter_now = ptx::ld_volatile(p.iter);
  const int parity = static_cast<int>(iter_now & 1u);
  int m = a.num_tokens;
  if (a.bound_m != nullptr) m = min(m, static_cast<int>(__ldg(a.bound_m)));
  m = min(m, p.max_tokens);
  trace(p, kTrDispatchStart);
  trace_block(p, kTrBlockDispatchStart);
  if constexpr (SEND) send_phase<kMode>(a, sm, parity, m, iter_now);
  if constexpr (SEND && RECV) __syncthreads();
  if constexpr (RECV) recv_phase<kMode>(a, sm, parity, iter_now);
  __syncthreads();
  trace_block(p, kTrBlockDispatchEnd);
}

template <bool SEND, bool RECV, int kMode>
__global__ void __launch_bounds__(kDispatchThreads, 1)
    dispatch_kernel(const __grid_constant__ DispatchArgs a) {
  extern __shared__ __align__(16) uint32_t dyn_smem[];
  dispatch_body<SEND, RECV, kMode>(a, dyn_smem);
}

// Several ranks that live on one device, run as one grid: blockIdx.y picks the
// rank.  Blocks of different ranks wait on one another, so the launch is
// cooperative to have them all resident.
template <bool SEND, bool RECV, int kMode>
__global__ void __launch_bounds__(kDispatchThreads, 1)
    dispatch_kernel_multi(const __grid_constant__ DispatchMulti m) {
  extern __shared__ __align__(16) uint32_t dyn_smem[];
  dispatch_body<SEND, RECV, kMode>(m.r[blockIdx.y], dyn_smem);
}

}  // namespace

size_t dispatch_smem_bytes(const A2AParams& p, int stage_tokens) {
  const size_t E = p.num_experts, P = static_cast<size_t>(p.world) * p.nle;
  const size_t words = 4 * E + (P + 1) + P + kMaxWorld + kRowCap;
  const size_t row = round_up<size_t>(static_cast<size_t>(p.hidden_bytes) + p.scale_bytes, 16);
  return round_up<size_t>(sizeof(uint32_t) * words, 16) + static_cast<size_t>(stage_tokens) * row;
}

int dispatch_stage_tokens(const A2AParams& p) {
  // Rows fetched from host memory per round: as many as fit into 64 KiB, at most 8.
  const size_t row = round_up<size_t>(static_cast<size_t>(p.hidden_bytes) + p.scale_bytes, 16);
  return static_cast<int>(std::min<size_t>(8, (64 * 1024) / row));
}

int dispatch_threads() { return kDispatchThreads; }

namespace {

// The instantiation that serves a launch.  The receive half only distinguishes lines from
// counters: the packed sends have no receive half of this kernel, and a quantised row is
// received like any other.
int mode_of(const DispatchArgs& a, bool send) {
  if (a.packed) return a.quantize ? kModePackedQuant : kModePacked;
  if (a.quantize) return send ? kModeQuant : kModeCounters;
  if (a.p.ll == 0) return kModeCounters;
  return (send && a.stage_tokens > 0) ? kModeLinesStaged : kModeLines;
}

template <template <bool, bool, int> class Pick>
const void* pick_kernel(bool send, bool recv, int mode) {
  // Only the combinations that exist are instantiated.
  if (send && recv) {
    switch (mode) {
      case kModeLines: return Pick<true, true, kModeLines>::fn();
      case kModeLinesStaged: return Pick<true, true, kModeLinesStaged>::fn();
      case kModeCounters: return Pick<true, true, kModeCounters>::fn();
      case kModeQuant: return Pick<true, true, kModeQuant>::fn();
      default: return nullptr;
    }
  }
  if (send) {
    switch (mode) {
      case kModeLines: return Pick<true, false, kModeLines>::fn();
      case kModeLinesStaged: return Pick<true, false, kModeLinesStaged>::fn();
      case kModeCounters: return Pick<true, false, kModeCounters>::fn();
      case kModeQuant: return Pick<true, false, kModeQuant>::fn();
      case kModePacked: return Pick<true, false, kModePacked>::fn();
      case kModePackedQuant: return Pick<true, false, kModePackedQuant>::fn();
      default: return nullptr;
    }
  }
  switch (mode) {
    case kModeLines: return Pick<false, true, kModeLines>::fn();
    case kModeCounters: return Pick<false, true, kModeCounters>::fn();
    default: return nullptr;
  }
}

template <bool SEND, bool RECV, int kMode>
struct SingleKernel {
  static const void* fn() { return reinterpret_cast<const void*>(&dispatch_kernel<SEND, RECV, kMode>); }
};
template <bool SEND, bool RECV, int kMode>
struct MultiKernel {
  static const void* fn() {
    return reinterpret_cast<const void*>(&dispatch_kernel_multi<SEND, RECV, kMode>);
  }
};

// Histograms of many experts and staged rows need more dynamic shared memory than a kernel
// gets by default.
cudaError_t allow_smem(const void* kernel, size_t smem) {
  if (smem <= 48 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(smem));
}

}  // namespace

cudaError_t launch_dispatch(const DispatchArgs& a, bool send, bool recv, int grid,
                            cudaStream_t stream) {
  const int mode = mode_of(a, send);
  const void* fn = pick_kernel<SingleKernel>(send, recv, mode);
  if (fn == nullptr) return cudaErrorInvalidValue;
  const size_t smem = dispatch_smem_bytes(a.p, mode == kModeLinesStaged ? a.stage_tokens : 0);
  const cudaError_t err = allow_smem(fn, smem);
  if (err != cudaSuccess) return err;
  void* params[] = {const_cast<DispatchArgs*>(&a)};
  return cudaLaunchKernel(fn, dim3(grid), dim3(kDispatchThreads), params, smem, stream);
}

cudaError_t launch_dispatch_multi(const DispatchMulti& args, int nranks, bool send, bool recv,
                                  int grid, cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxLocalRanks) return cudaErrorInvalidValue;
  // All ranks of an emulated world run one instantiation: the mode of rank 0, which the
  // others must share.
  const int mode = mode_of(args.r[0], send);
  int stage_tokens = 0;
  for (int r = 0; r < nranks; ++r) {
    if (mode_of(args.r[r], send) != mode) return cudaErrorInvalidValue;
    stage_tokens = std::max(stage_tokens, args.r[r].stage_tokens);
  }
  const void* fn = pick_kernel<MultiKernel>(send, recv, mode);
  if (fn == nullptr) return cudaErrorInvalidValue;
  const size_t smem = dispatch_smem_bytes(args.r[0].p, mode == kModeLinesStaged ? stage_tokens : 0);
  const cudaError_t err = allow_smem(fn, smem);
  if (err != cudaSuccess) return err;
  void* params[] = {const_cast<DispatchMulti*>(&args)};
  return cudaLaunchCooperativeKernel(fn, dim3(grid, nranks), dim3(kDispatchThreads), params, smem,
                                     stream);
}

}  // namespace pplx
