// Decode-sized dispatch: a handful of tokens per rank, where latency is everything.
//
// Capability parity: the per-token protocol of the reference's intranode dispatch
// (intranode_dispatch.cu:187-223) serves every batch size with global atomics and three
// grid-wide barriers; this kernel is the specialisation for objects of at most
// PPLX_B200_TINY_MAX_TOKENS tokens and removes every step that is not a memory round trip
// the data needs anyway:
//
//  * No histogram, no prefix sums, no counts exchange, no global atomics.  Token number o of
//    a source owns a fixed group of S = min(top-k, local experts) slots in the source's
//    staging region at every destination; its j-th row for a destination goes to slot
//    o * S + j.
//  * One HEADER line per (destination, source, token): how many rows the token sends there
//    and, per row, (k, local expert).  A token without rows for a destination -- and a token
//    slot beyond bound_m -- still writes its (empty) header, so the receiver knows when it
//    has seen everything without knowing any count in advance.
//  * Header and rows are flag-in-data lines (core/ll128.cuh): the sender never waits, the
//    receiver polls the data itself.  Headers exist twice, selected by the parity of the
//    iteration counter, because a rank may be one dispatch ahead of a peer (see
//    a2a_params.h); rows need no second copy for the reason given there.
//  * The rows of one token are sent by several blocks (each derives the token's table from
//    the same indices), so a single token uses as many SMs as it has rows.
//  * Every receiving block reads ALL headers (a few kilobytes of local memory) and derives
//    the same table from them: entry (source, token, j) of local expert e takes the output
//    row equal to the number of earlier entries of e, in (source, token, j) order.  No
//    block therefore needs anything from another block of its own grid: no cursor atomics,
//    no last-block epilogue, and the rows -- split into line ranges when there are more
//    warps than rows -- are copied by all warps of the grid.
//
// Send: 1 cold read of `indices`, then header and row lines.  Receive: poll the headers,
// a few hundred cycles of shared-memory bookkeeping, poll and copy the rows.
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

constexpr int kTinyThreads = 512;
constexpr int kTinyWarps = kTinyThreads / 32;
constexpr int kTinyMaxTopk = 32;
constexpr int kTinyMaxSlots = 29;      // rows of a token per destination: words 1..29 of a header
constexpr int kTinyMaxEntries = 2048;  // world * tokens per sender * S
constexpr int kTinyMaxLocalExperts = 1024;
constexpr uint32_t kNoEntry = 0xffffffffu;

struct TinySmem {
  // send side: the table of the token this block is sending
  uint32_t dst[kTinyMaxTopk];    // destination rank of entry k, or kNoEntry
  uint32_t le[kTinyMaxTopk];     // local expert there
  uint32_t j[kTinyMaxTopk];      // ordinal among the token's rows for that destination
  uint32_t tbl[kMaxWorld * 32];  // [dst][j] -> k | le << 16
  // receive side
  uint32_t entry[kTinyMaxEntries];  // [(source, token), j] -> k | le << 16, or kNoEntry
  uint32_t row[kTinyMaxEntries];    // output row of that entry within its expert
  uint16_t list[kTinyMaxEntries];   // the valid entries, compacted
  uint32_t cnt[kTinyMaxLocalExperts];  // rows assigned so far per local expert
  uint32_t valid;                   // how many
};

__device__ __forceinline__ void stamp(const A2AParams& p, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.trace[slot] = ptx::globaltimer_ns();
}

__device__ __forceinline__ uint8_t* header_line(const A2AParams& p, int owner, int parity, int src,
                                                int tokens_per_sender, int o) {
  return p.peer[owner] + p.off_tiny_hdr +
         ((static_cast<size_t>(parity) * p.world + src) * tokens_per_sender + o) * ll::kLineBytes;
}

// In how many line ranges a row of `lines` lines is split so that `rows` rows keep about
// `warps` warps busy (a warp instruction moves four lines).
__device__ __forceinline__ int split_for(int rows, int warps, int lines) {
  int split = 1;
  while (split < 16 && split * 2 * rows <= warps && lines >= split * 2 * 4) split *= 2;
  return split;
}

__device__ __forceinline__ void tiny_send(const DispatchArgs& a, TinySmem& sm, int parity,
                                          uint32_t iter_now) {
  const A2AParams& p = a.p;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int topk = p.topk;
  const int S = min(topk, p.nle);
  const int dp_rank = p.rank % p.dp_size;
  const int tokens_per_sender = ceil_div<int>(p.max_tokens, p.dp_size);
  const uint64_t flag = ll::kDispatchTag | static_cast<uint64_t>(iter_now + 1u);
  const int nscale = p.scale_bytes >> 2;
  const int limit = min(a.num_tokens, p.max_tokens);

  if (blockIdx.x == 0 && tid == 0) {
    const uint32_t started = *p.comb_iter;
    if (started != iter_now)
      report_failure(p.status, kOutOfOrder, kPhaseDispatchCounts, 0, iter_now, started, p.rank);
    *p.comb_iter = started + 1u;
  }

  // Blocks per token: the rows k with k % bpt == part are this block's.
  const int bpt = max(1, min(topk, static_cast<int>(gridDim.x) / tokens_per_sender));
  const int send_units = tokens_per_sender * bpt;
  for (int su = blockIdx.x; su < send_units; su += gridDim.x) {
    const int o = su / bpt;
    const int part = su - o * bpt;
    const int i = o * p.dp_size + dp_rank;  // every token slot, with or without a token in it
    // The indices are fetched before bound_m is known (both reads are cold): a row of
    // `indices` exists for every i < num_tokens.
    uint32_t e = kNoEntry;
    if (tid < topk && i < limit) e = __ldg(a.indices + static_cast<size_t>(i) * topk + tid);
    int m = limit;
    if (a.bound_m != nullptr) m = min(m, static_cast<int>(__ldg(a.bound_m)));
    const bool has = i < m;
    if (!has && part != 0) continue;  // an empty slot is its header only (uniform per block)
    if (tid < topk) {
      uint32_t dst = kNoEntry, le = 0;
      if (has) {
        if (e < static_cast<uint32_t>(p.num_experts)) {
          dst = e / p.nle;
          le = e - dst * p.nle;
        } else if (p.debug_checks) {
          report_failure(p.status, kBadExpert, kPhaseDispatchCounts, i, p.num_experts, e, p.rank);
        }
      }
      sm.dst[tid] = dst;
      sm.le[tid] = le;
    }
    __syncthreads();
    if (tid < topk) {
      const uint32_t dst = sm.dst[tid];
      uint32_t j = 0;
      for (int k2 = 0; k2 < tid; ++k2) j += sm.dst[k2] == dst;
      if (dst != kNoEntry && j >= static_cast<uint32_t>(S)) {
        // More rows for one destination than it owns experts: the token names an expert
        // twice.  The surplus row is dropped and reported.
        if (part == 0)
          report_failure(p.status, kSlotOverflow, kPhaseDispatchPayload, dst, S, j, p.rank);
        j = kNoEntry;
      }
      sm.j[tid] = j;
      if (dst != kNoEntry && j != kNoEntry) sm.tbl[dst * 32 + j] = tid | (sm.le[tid] << 16);
    }
    __syncthreads();
    stamp(p, kTrDispatchHist);

    // Headers: one line per destination; a warp instruction writes four of them.
    if (part == 0 && warp == kTinyWarps - 1) {
      const int c = lane & 7;
      for (int d0 = 0; d0 < p.world; d0 += 4) {
        const int d = d0 + (lane >> 3);
        if (d < p.world) {
          uint32_t n = 0;
          for (int k2 = 0; k2 < topk; ++k2)
            n += sm.dst[k2] == static_cast<uint32_t>(d) && sm.j[k2] != kNoEntry;
          uint32_t w[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int word = 4 * c + t;  // word 0: n; word 1 + j: row j
            uint32_t v = 0;
            if (word == 0) v = n;
            else if (static_cast<uint32_t>(word - 1) < n) v = sm.tbl[d * 32 + word - 1];
            w[t] = v;
          }
          const uint64_t lo = static_cast<uint64_t>(w[0]) | (static_cast<uint64_t>(w[1]) << 32);
          const uint64_t hi = c == 7 ? flag
                                     : static_cast<uint64_t>(w[2]) | (static_cast<uint64_t>(w[3]) << 32);
          ll::st16(header_line(p, d, parity, p.rank, tokens_per_sender, o) + c * 16, lo, hi);
        }
      }
    }
    stamp(p, kTrDispatchPosted);

    // Rows: units of (k, line range) over the warps of the block.
    if (has) {
      const int mine = (topk - part + bpt - 1) / bpt;
      const int split = split_for(mine, kTinyWarps, p.ll_x_lines);
      const uint8_t* src = a.x + static_cast<int64_t>(i) * a.x_stride_row;
      for (int unit = warp; unit < mine * split; unit += kTinyWarps) {
        const int k = part + (unit / split) * bpt;
        const int c = unit % split;
        const uint32_t dst = sm.dst[k];
        const uint32_t j = sm.j[k];
        if (dst == kNoEntry || j == kNoEntry) continue;
        uint8_t* slot = p.peer[dst] + p.off_ll_disp_stage +
                        (static_cast<size_t>(p.rank) * p.region_slots + o * S + j) * p.ll_slot_bytes;
        const int l0 = (c * p.ll_x_lines) / split;
        const int l1 = ((c + 1) * p.ll_x_lines) / split;
        ll::warp_send_lines(slot, src, p.hidden_bytes, l0, l1, flag, lane);
        if (c == split - 1) {
          const uint32_t trailer[4] = {static_cast<uint32_t>(i), static_cast<uint32_t>(k), sm.le[k],
                                       static_cast<uint32_t>(p.rank)};
          const float* ssrc =
              nscale > 0 ? a.x_scale + static_cast<int64_t>(i) * a.x_scale_stride_row : nullptr;
          ll::warp_send_meta(slot + p.ll_x_lines * ll::kLineBytes, p.ll_meta_lines, trailer, ssrc,
                             a.x_scale_stride_col, nscale, flag, lane);
        }
      }
    }
    stamp(p, kTrDispatchStored);
    __syncthreads();  // the tables are rewritten for the block's next unit
  }
}

// Reads every header addressed to this rank into sm.entry.  A header that never arrives is
// reported and treated as empty, so that the kernel ends.
__device__ __forceinline__ void read_headers(const A2AParams& p, TinySmem& sm, int parity,
                                             uint64_t flag, const WaitCtx& w) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int S = min(p.topk, p.nle);
  const int tokens_per_sender = ceil_div<int>(p.max_tokens, p.dp_size);
  const int headers = p.world * tokens_per_sender;  // h = source * tokens_per_sender + token
  const uint8_t* base = header_line(p, p.rank, parity, 0, tokens_per_sender, 0);
  const int c = lane & 7, g = lane >> 3;
  for (int h0 = warp * 4; h0 < headers; h0 += kTinyWarps * 4) {
    const int h = h0 + g;
    uint64_t lo = 0, hi = 0;
    ll::Poll poll(w, kPhaseDispatchCounts, static_cast<uint32_t>(h0 / tokens_per_sender));
    bool ok = true;
    while (true) {
      bool ready = true;
      if (h < headers) {
        ll::ld16(base + static_cast<size_t>(h) * ll::kLineBytes + c * 16, lo, hi);
        ready = c != 7 || hi == flag;
      }
      if (__all_sync(0xffffffffu, ready)) break;
      if (!poll.again(lane, flag, hi)) {
        ok = false;
        break;
      }
    }
    uint32_t n = __shfl_sync(0xffffffffu, static_cast<uint32_t>(lo), lane & ~7);
    if (!ok) n = 0;
    if (n > static_cast<uint32_t>(S)) {
      if (c == 0)
        report_failure(p.status, kBadToken, kPhaseDispatchCounts, h / tokens_per_sender, S, n,
                       p.rank);
      n = 0;
    }
    if (h < headers) {
      const uint32_t mine[4] = {static_cast<uint32_t>(lo), static_cast<uint32_t>(lo >> 32),
                                static_cast<uint32_t>(hi), static_cast<uint32_t>(hi >> 32)};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int j = 4 * c + t - 1;  // word 1 + j of the line
        if (j >= 0 && j < S && (c < 7 || t < 2))
          sm.entry[h * S + j] = static_cast<uint32_t>(j) < n ? mine[t] : kNoEntry;
      }
    }
  }
}

// From sm.entry: the output row of every entry (the number of earlier entries of the same
// local expert, in (source, token, j) order), the compacted list of valid entries, and -- block
// 0 -- the totals.  One warp walks the entries 32 at a time; lanes that name the same expert find
// each other with a match instruction, so the cost does not depend on how many experts a rank
// owns.  Block-wide call.
__device__ __forceinline__ void assign_rows(const DispatchArgs& a, TinySmem& sm, int entries) {
  const A2AParams& p = a.p;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  for (int le = tid; le < p.nle; le += blockDim.x) sm.cnt[le] = 0;
  __syncthreads();
  if (warp == 0) {
    uint32_t nvalid = 0;
    for (int e0 = 0; e0 < entries; e0 += 32) {
      const int e = e0 + lane;
      const uint32_t v = e < entries ? sm.entry[e] : kNoEntry;
      const uint32_t le = v >> 16;
      // An entry that names an expert or a k this rank does not have is dropped here.
      const bool hit = v != kNoEntry && le < static_cast<uint32_t>(p.nle) &&
                       (v & 0xffffu) < static_cast<uint32_t>(p.topk);
      if (v != kNoEntry && !hit)
        report_failure(p.status, kBadToken, kPhaseDispatchPayload, 0, p.nle, le, p.rank);
      const uint32_t active = __ballot_sync(0xffffffffu, hit);
      uint32_t same = 0, base = 0;
      if (hit) {
        same = __match_any_sync(active, le);
        base = sm.cnt[le];
        sm.row[e] = base + __popc(same & lt);
        sm.list[nvalid + __popc(active & lt)] = static_cast<uint16_t>(e);
      }
      __syncwarp();  // every lane of a group has read the count before its first lane moves it on
      if (hit && (same & lt) == 0u) sm.cnt[le] = base + __popc(same);
      __syncwarp();
      nvalid += __popc(active);
    }
    if (lane == 0) sm.valid = nvalid;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int le = tid; le < p.nle; le += blockDim.x) {
      const uint32_t total = sm.cnt[le];
      a.out_num_tokens[le] = static_cast<int32_t>(total);
      p.recv_count[le] = min(total, static_cast<uint32_t>(p.cap));
    }
  }
}

__device__ __forceinline__ void tiny_recv(const DispatchArgs& a, TinySmem& sm, int parity,
                                          uint32_t iter_now) {
  const A2AParams& p = a.p;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int S = min(p.topk, p.nle);
  const int tokens_per_sender = ceil_div<int>(p.max_tokens, p.dp_size);
  const uint64_t flag = ll::kDispatchTag | static_cast<uint64_t>(iter_now + 1u);
  const WaitCtx w{p.status, p.timeout_ns, static_cast<uint32_t>(p.rank)};
  const int nscale = p.scale_bytes >> 2;
  const int entries = p.world * tokens_per_sender * S;

  read_headers(p, sm, parity, flag, w);
  __syncthreads();
  stamp(p, kTrDispatchCounts);
  assign_rows(a, sm, entries);
  __syncthreads();
  stamp(p, kTrDispatchLayout);

  const int valid = static_cast<int>(sm.valid);
  const int gwarps = gridDim.x * kTinyWarps;
  const int split = split_for(valid, gwarps, p.ll_x_lines);
  for (int unit = blockIdx.x * kTinyWarps + warp; unit < valid * split; unit += gwarps) {
    const int e = sm.list[unit / split];
    const int c = unit % split;
    const uint32_t v = sm.entry[e];
    const uint32_t k = v & 0xffffu, le = v >> 16;
    const uint32_t row = sm.row[e];
    const int h = e / S, j = e - h * S;
    const int s = h / tokens_per_sender, o = h - s * tokens_per_sender;
    if (row >= static_cast<uint32_t>(p.cap)) {
      if (lane == 0 && c == 0)
        report_failure(p.status, kRowOverflow, kPhaseDispatchPayload, s, p.cap, row, p.rank);
      continue;
    }
    const uint8_t* slot = p.peer[p.rank] + p.off_ll_disp_stage +
                          (static_cast<size_t>(s) * p.region_slots + o * S + j) * p.ll_slot_bytes;
    uint8_t* dst = a.out_x + le * a.out_x_stride_e + static_cast<int64_t>(row) * a.out_x_stride_row;
    ll::Poll rows(w, kPhaseDispatchPayload, static_cast<uint32_t>(s));
    const int l0 = (c * p.ll_x_lines) / split;
    const int l1 = ((c + 1) * p.ll_x_lines) / split;
    if (!ll::warp_recv_lines(dst, slot, p.hidden_bytes, l0, l1, flag, lane, rows)) continue;
    if (c != split - 1) continue;
    if (nscale > 0) {
      uint32_t trailer[4];
      float* sdst = a.out_scale + le * a.out_scale_stride_e +
                    static_cast<int64_t>(row) * a.out_scale_stride_row;
      if (!ll::warp_recv_meta(slot + p.ll_x_lines * ll::kLineBytes, p.ll_meta_lines, sdst,
                              a.out_scale_stride_col, nscale, flag, lane, rows, trailer))
        continue;
    }
    if (lane == 0) {
      uint2 rs;
      rs.x = static_cast<uint32_t>(s) | (k << 16);
      rs.y = static_cast<uint32_t>(o * p.dp_size + s % p.dp_size);
      p.row_src[static_cast<size_t>(le) * p.cap + row] = rs;
    }
  }
  stamp(p, kTrDispatchCopied);
}

template <bool SEND, bool RECV>
__device__ __forceinline__ void tiny_body(const DispatchArgs& a) {
  __shared__ TinySmem sm;
  const A2AParams& p = a.p;
  const uint32_t iter_now = ptx::ld_volatile(p.iter);
  const int parity = static_cast<int>(iter_now & 1u);
  stamp(p, kTrDispatchStart);
  if (p.trace != nullptr && threadIdx.x == 0 && blockIdx.x < kTraceBlocks)
    p.trace[kTrBlockDispatchStart + blockIdx.x] = ptx::globaltimer_ns();
  if constexpr (SEND) tiny_send(a, sm, parity, iter_now);
  stamp(p, kTrDispatchSignalled);
  if constexpr (RECV) tiny_recv(a, sm, parity, iter_now);
  __syncthreads();
  stamp(p, kTrDispatchEnd);
  if (p.trace != nullptr && threadIdx.x == 0 && blockIdx.x < kTraceBlocks)
    p.trace[kTrBlockDispatchEnd + blockIdx.x] = ptx::globaltimer_ns();
}

template <bool SEND, bool RECV>
__global__ void __launch_bounds__(kTinyThreads, 1)
    dispatch_tiny_kernel(const __grid_constant__ DispatchArgs a) {
  tiny_body<SEND, RECV>(a);
}

template <bool SEND, bool RECV>
__global__ void __launch_bounds__(kTinyThreads, 1)
    dispatch_tiny_kernel_multi(const __grid_constant__ DispatchMulti m) {
  tiny_body<SEND, RECV>(m.r[blockIdx.y]);
}

template <bool kMulti>
const void* tiny_fn(bool send, bool recv) {
  if constexpr (kMulti) {
    if (send && recv) return reinterpret_cast<const void*>(&dispatch_tiny_kernel_multi<true, true>);
    if (send) return reinterpret_cast<const void*>(&dispatch_tiny_kernel_multi<true, false>);
    return reinterpret_cast<const void*>(&dispatch_tiny_kernel_multi<false, true>);
  } else {
    if (send && recv) return reinterpret_cast<const void*>(&dispatch_tiny_kernel<true, true>);
    if (send) return reinterpret_cast<const void*>(&dispatch_tiny_kernel<true, false>);
    return reinterpret_cast<const void*>(&dispatch_tiny_kernel<false, true>);
  }
}

}  // namespace

bool dispatch_tiny_supports(const A2AParams& p) {
  const int S = min(p.topk, p.nle);
  const int tokens_per_sender = ceil_div<int>(p.max_tokens, p.dp_size);
  return p.topk <= kTinyMaxTopk && p.world <= kMaxWorld && S <= kTinyMaxSlots &&
         p.nle <= kTinyMaxLocalExperts &&
         p.world * tokens_per_sender * S <= kTinyMaxEntries;
}

int dispatch_tiny_grid(const A2AParams& p, int limit) {
  // One block per (token slot, row) on the sending side; the receiving side spreads its rows
  // over whatever grid there is.
  const int tokens_per_sender = ceil_div<int>(p.max_tokens, p.dp_size);
  int grid = tokens_per_sender * p.topk;
  grid = grid < 4 ? 4 : grid;
  return grid > limit ? limit : grid;
}

cudaError_t launch_dispatch_tiny(const DispatchArgs& a, bool send, bool recv, int grid,
                                 cudaStream_t stream) {
  void* params[] = {const_cast<DispatchArgs*>(&a)};
  return cudaLaunchKernel(tiny_fn<false>(send, recv), dim3(grid), dim3(kTinyThreads), params, 0,
                          stream);
}

cudaError_t launch_dispatch_tiny_multi(const DispatchMulti& args, int nranks, bool send, bool recv,
                                       int grid, cudaStream_t stream) {
  if (nranks < 1 || nranks > kMaxLocalRanks) return cudaErrorInvalidValue;
  void* params[] = {const_cast<DispatchMulti*>(&args)};
  return cudaLaunchCooperativeKernel(tiny_fn<true>(send, recv), dim3(grid, nranks),
                                     dim3(kTinyThreads), params, 0, stream);
}

}  // namespace pplx
