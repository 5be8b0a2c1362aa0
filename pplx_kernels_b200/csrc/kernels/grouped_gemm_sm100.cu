// Grouped expert GEMM for sm_100a: for every local expert e with counts[e] rows,
//   out[e, :counts[e], :] = act(x[e, :counts[e], :] @ w[e]^T)
// with bf16 operands, fp32 accumulation in tensor memory and a bf16 result.
// `act` is the identity, or SwiGLU when w[e] stacks a gate and an up projection
// ([2 * I, K]) and the result has I columns: silu(x @ gate^T) * (x @ up^T).
//
// The reference contains no GEMM; this kernel serves the fused MoE layer that
// goes beyond it.  Design (one CTA per SM, persistent over tiles):
//
//   warp 0      TMA producer: cp.async.bulk.tensor tile loads of x and w into a
//               ring of 128-byte-swizzled shared-memory stages (no multicast)
//   warp 1      one elected thread issues tcgen05.mma (M=128, N=256, K=16 per
//               instruction) into one of two 256-column accumulators in tensor
//               memory, and tcgen05.commit to hand stages and accumulators on
//   warp 2      allocates / frees the 512 tensor-memory columns
//   warps 4-7   epilogue: tcgen05.ld of the finished accumulator, activation,
//               bf16 conversion, masked 16-byte global stores; overlaps with the
//               MMAs of the next tile through the second accumulator
//
// With kTwoCta the kernel runs as clusters of two CTAs that share one 256-row tile
// (tcgen05 cta_group::2): each CTA loads its own 128 rows of A and HALF of the
// weight tile, the leader CTA issues M = 256 MMAs that read both CTAs' shared
// memory, and each CTA keeps and drains the accumulator of its own 128 rows.
// Per SM that halves the weight traffic into shared memory and the shared-memory
// reads per MMA, which is what limits the one-CTA form.  No TMA multicast is
// involved: the two CTAs load different data; only barrier arrivals
// (tcgen05.commit) are delivered to both CTAs.
//
// Tiles are (expert, 256-column block, 128-row block) with the row block varying
// fastest, so CTAs that run at the same time share a weight tile in L2.  The
// row counts are read on the device, so the launch is graph-capturable and does
// no work for empty experts.
//
// Two template switches turn the same pipeline into the compute+collective
// kernels of the fused MoE layer:
//
//   kFromStaging   the A operand is read by TMA straight out of the dispatch
//                  staging arena that PEERS fill with P2P stores (packed send:
//                  rows grouped by local expert, then by source rank, dense).
//                  Arrival is counted per (expert, source): before a tile the
//                  producer warp waits (ld.acquire.sys, then fence.proxy.async)
//                  only for the sources whose rows the tile covers, so the expert
//                  GEMM starts tile by tile as tokens land and the receive-side
//                  copy of dispatch disappears.  The epilogue also records
//                  (source, token, k) of every row for combine.
//   kToPeers       the epilogue does not write a local result: every output row
//                  is stored into the combine staging of the token's home rank(s)
//                  over NVLink, followed once per tile by one system-scope fence
//                  and relaxed adds on the tokens' arrival counters.  The
//                  combine send kernel and the expert_y round trip disappear.
//
// Every mbarrier wait is bounded: when one runs out the CTA raises a shared
// abort flag, all roles leave their loops, in-flight TMA loads are drained,
// tensor memory is freed and the kernel returns with *status = 1.
#include <algorithm>

#include <cuda.h>
#include <cuda_bf16.h>
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
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kStages = 4;      // one CTA per tile: 16 KiB of A + 32 KiB of B per stage
constexpr int kStages2 = 6;     // CTA pair: 16 KiB of A + 16 KiB of B per stage and CTA
constexpr int kMaxStages = 6;
constexpr int kThreads = 256;
constexpr int kTmemCols = 512;
constexpr uint32_t kABytes = kBlockM * kBlockK * 2;  // 16 KiB
constexpr uint32_t kBBytes = kBlockN * kBlockK * 2;  // 32 KiB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kStageBytes2 = kABytes + kBBytes / 2;
constexpr uint64_t kWaitLimitNs = 2000000000ull;     // 2 s per wait
constexpr int kMaxExperts = 1024;

constexpr uint32_t kNoSignal = 0xffffffffu;

// Peer-storing epilogue: an epilogue thread owns one ROW of the tile, so storing straight from
// registers would send 32 separate 16-byte pieces per instruction over NVLink.  Each epilogue
// warp therefore passes 64 columns at a time through a [32 rows][128 B + 16 B pad] buffer in
// shared memory and writes them out as 128-byte row segments (eight lanes per row).
constexpr int kOutStageRowBytes = 144;
struct PeerStage {
  uint8_t rows[4][32][kOutStageRowBytes];   // one buffer per epilogue warp
  unsigned long long row_off[2][kBlockM];   // arena offset of each tile row's combine slot
};

// One tensor map of the weights per candidate tile width (the TMA box height is
// fixed in the map); the kernel picks the width once it knows the real row counts.
struct WeightMaps {
  CUtensorMap m[kNumTileWidths];
};

struct SharedControl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t pad[2];
  uint32_t sig_token[2][kBlockM];  // kToPeers: token of each tile row, per accumulator
  uint32_t sig_group[2][kBlockM];  //           first rank of the token's DP group
};

// Rows of A that share a weight matrix: one group per local expert.  With
// kFromStaging the rows of all experts sit back to back in one plane of A and
// a_row0 is the expert's first row there.
struct GroupTable {
  uint32_t* tile_start;  // [G + 1] first tile of each group
  uint32_t* rows;        // [G] valid rows
  uint32_t* a_row0;      // [G] first row inside the A plane
  uint32_t* out_row0;    // [G] first row inside the output plane
  uint32_t* src_rows;    // kFromStaging: [G][world] rows that each source sends to the group,
                         // or null when the table does not fit (then a tile waits for all
                         // sources of its expert)
};

struct TileCoord {
  int group;
  int m_blk;
  int n_blk;
  int rows;      // valid rows of the group
  int a_plane;   // dim-2 coordinate of A
  int a_row0;
  int w_plane;   // expert whose weights apply
  int out_row0;
};

// Tiles of one group are ordered (n_blk, m_blk) with m_blk fastest.
template <bool kFromStaging>
__device__ __forceinline__ TileCoord locate_tile(const GroupTable& gt, int num_groups,
                                                 const A2AParams& p, uint32_t t, int tile_m) {
  TileCoord c;
  c.group = find_group(gt.tile_start, num_groups, t);
  c.rows = static_cast<int>(gt.rows[c.group]);
  const int m_tiles = ceil_div<int>(c.rows, tile_m);
  const uint32_t rem = t - gt.tile_start[c.group];
  c.n_blk = static_cast<int>(rem / m_tiles);
  c.m_blk = static_cast<int>(rem - static_cast<uint32_t>(c.n_blk) * m_tiles);
  c.a_row0 = static_cast<int>(gt.a_row0[c.group]);
  c.out_row0 = static_cast<int>(gt.out_row0[c.group]);
  c.w_plane = c.group;
  c.a_plane = kFromStaging ? 0 : c.group;
  (void)p;
  return c;
}

__device__ __forceinline__ float silu(float v) { return v / (1.0f + __expf(-v)); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <bool SWIGLU, bool kFromStaging, bool kToPeers, bool kTwoCta>
__global__ void __launch_bounds__(kThreads, 1)
    grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ WeightMaps wmaps,
                        const __grid_constant__ GroupedGemmArgs g) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // Stage ring first (1024-byte aligned tiles), control block and tile table after.
  uint8_t* stages = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  constexpr int kNumStages = kTwoCta ? kStages2 : kStages;
  constexpr uint32_t kStageStride = kTwoCta ? kStageBytes2 : kStageBytes;
  SharedControl* ctl = reinterpret_cast<SharedControl*>(stages + kNumStages * kStageStride);
  // A CTA pair works on one tile of 256 rows; this CTA owns rows [128 * cta_rank, +128).
  const uint32_t cta_rank = kTwoCta ? tc::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0u;
  const int tile_m = kTwoCta ? 2 * kBlockM : kBlockM;
  const uint32_t worker = kTwoCta ? blockIdx.x >> 1 : blockIdx.x;   // tile-loop index
  const uint32_t workers = kTwoCta ? gridDim.x >> 1 : gridDim.x;
  const A2AParams& p = g.a2a;
  const int num_groups = g.num_experts;
  GroupTable gt;
  gt.tile_start = reinterpret_cast<uint32_t*>(ctl + 1);  // [G + 1]
  gt.rows = gt.tile_start + num_groups + 1;
  gt.a_row0 = gt.rows + num_groups;
  gt.out_row0 = gt.a_row0 + num_groups;
  gt.src_rows = (kFromStaging && g.src_table != 0) ? gt.out_row0 + num_groups : nullptr;
  // (kToPeers only) staging of the peer-storing epilogue, behind the tables, 16-byte aligned.
  PeerStage* peer_stage = reinterpret_cast<PeerStage*>(
      (reinterpret_cast<uintptr_t>(gt.out_row0 + num_groups) + 15) & ~static_cast<uintptr_t>(15));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  const int num_kb = ceil_div<int>(g.k, kBlockK);

  // ---- set-up ---------------------------------------------------------------
  if (tid == 0) ctl->abort_flag = 0;
  int parity = 0;
  if constexpr (kFromStaging || kToPeers) parity = static_cast<int>(ptx::ld_volatile(p.iter) & 1u);
  if constexpr (kFromStaging) {
    // Role of the dispatch receive phase: learn how many rows every source sends
    // to every local expert, lay the rows out, publish the per-expert totals.
    for (int le = tid; le < num_groups; le += blockDim.x) gt.rows[le] = 0;
    __syncthreads();
    const WaitCtx w{p.status, p.timeout_ns, static_cast<uint32_t>(p.rank)};
    const uint32_t* all = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.off_counts_all) +
                          static_cast<size_t>(parity) * p.world * p.num_experts;
    for (int idx = tid; idx < p.world * p.nle; idx += blockDim.x) {
      const int src = idx / p.nle;
      const int le = idx - src * p.nle;
      uint32_t v = 0;
      const bool ok = wait_until(all + static_cast<size_t>(src) * p.num_experts + p.rank * p.nle + le,
                                 PredNonZero{}, v, w, kPhaseDispatchCounts, src, 1u);
      if (!ok) ctl->abort_flag = 1;
      if (ok && v > 1u) atomicAdd(&gt.rows[le], v - 1u);
      if (gt.src_rows != nullptr) gt.src_rows[le * p.world + src] = (ok && v > 1u) ? v - 1u : 0u;
    }
    __syncthreads();
    for (int le = tid; le < num_groups; le += blockDim.x) {
      uint32_t first = 0;
      for (int l2 = 0; l2 < le; ++l2) first += gt.rows[l2];
      gt.a_row0[le] = first;
      gt.out_row0[le] = 0;
      const uint32_t rows = min(gt.rows[le], static_cast<uint32_t>(p.cap));
      gt.tile_start[le] = static_cast<uint32_t>(ceil_div<int>(static_cast<int>(rows), tile_m));
      if (blockIdx.x == 0) {
        if (g.out_num_tokens != nullptr) g.out_num_tokens[le] = static_cast<int32_t>(gt.rows[le]);
        p.recv_count[le] = rows;
      }
    }
    __syncthreads();
    for (int le = tid; le < num_groups; le += blockDim.x) gt.rows[le] = min(gt.rows[le], static_cast<uint32_t>(p.cap));
  } else {
    for (int e = tid; e < num_groups; e += blockDim.x) {
      const int rows = min(max(g.counts[e], 0), g.rows_per_expert);
      gt.rows[e] = static_cast<uint32_t>(rows);
      gt.a_row0[e] = 0;
      gt.out_row0[e] = 0;
      gt.tile_start[e] = static_cast<uint32_t>(ceil_div<int>(rows, tile_m));
    }
  }
  if constexpr (kToPeers) {
    if (blockIdx.x == 0) {
      // Role of the combine send phase's first block: the dispatch that produced
      // these rows is over on this rank, so clear its flag set and move on.
      uint32_t* counts = reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_counts) +
                         a2a_counts_index(p, parity, 0, 0);
      uint32_t* arrived =
          reinterpret_cast<uint32_t*>(p.peer[p.rank] + p.off_arrived) + parity * p.world;
      for (int q = tid; q < p.world * p.nle; q += blockDim.x) counts[q] = 0;
      if (tid < p.world) arrived[tid] = 0;
      reset_packed_flags(p, parity);
      __syncthreads();
      if (tid == 0) *p.iter = *p.iter + 1u;
    }
  }
  if (tid == 0) {
    for (int s = 0; s < kNumStages; ++s) {
      tc::mbar_init(&ctl->full[s], 1);
      tc::mbar_init(&ctl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&ctl->tmem_full[b], 1);
      tc::mbar_init(&ctl->tmem_empty[b], kTwoCta ? 8 : 4);  // epilogue warps of the tile
    }
    tc::fence_mbar_init();
    tc::tma_prefetch_desc(&tmap_a);
  }
  __syncthreads();
  if (warp == 0) warp_exclusive_scan_smem(gt.tile_start, num_groups, lane, true);
  if (warp == 2) {
    if constexpr (kTwoCta) {
      tc::tmem_alloc_2cta(&ctl->tmem_base, kTmemCols);
      tc::tmem_relinquish_2cta();
    } else {
      tc::tmem_alloc(&ctl->tmem_base, kTmemCols);
      tc::tmem_relinquish();
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  // The peer must see initialised barriers before anything arrives on them remotely.
  if constexpr (kTwoCta) tc::cluster_sync();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  // Tile width.  gt.tile_start holds the prefix of ROW blocks per expert; with the
  // real total the width that minimises (waves of tiles) x (time of one tile) is
  // chosen among the candidates the host prepared -- every CTA computes the same.
  // The B tile is two halves of half_n weight rows each (gate and up rows for
  // SwiGLU, consecutive rows otherwise); the accumulator is 2 * half_n columns wide.
  const uint32_t total_m_tiles = gt.tile_start[num_groups];
  int width_idx = 0;
  {
    uint64_t best = ~0ull;
    for (int i = 0; i < kNumTileWidths; ++i) {
      const int half = g.widths[i];
      if (half <= 0) continue;
      const uint32_t nb = ceil_div<uint32_t>(g.n_out, (SWIGLU ? 1 : 2) * half);
      const uint64_t waves = ceil_div<uint64_t>(static_cast<uint64_t>(total_m_tiles) * nb, workers);
      const uint64_t cost = waves * static_cast<uint64_t>(half + (kTwoCta ? 40 : 88));
      if (cost < best) {
        best = cost;
        width_idx = i;
      }
    }
  }
  const CUtensorMap& tmap_b = wmaps.m[width_idx];
  const int half_n = g.widths[width_idx];
  const int tile_n = 2 * half_n;
  const uint32_t b_half_bytes = static_cast<uint32_t>(half_n) * kBlockK * 2;
  // Bytes that complete one stage: both B halves from this CTA, or (pair) A and one
  // B half from each of the two CTAs, all counted on the leader's barrier.
  const uint32_t stage_tx_bytes = kTwoCta ? 2 * (kABytes + b_half_bytes) : kABytes + 2 * b_half_bytes;
  const int out_cols_per_tile = SWIGLU ? half_n : tile_n;
  const int n_blocks = ceil_div<int>(g.n_out, out_cols_per_tile);
  __syncthreads();
  for (int i = tid; i <= num_groups; i += blockDim.x) gt.tile_start[i] *= static_cast<uint32_t>(n_blocks);
  __syncthreads();
  const uint32_t total_tiles = gt.tile_start[num_groups];
  if (warp == 0 && lane == 0) tc::tma_prefetch_desc(&tmap_b);

  // ---- roles ----------------------------------------------------------------
  if (warp == 0) {
    if (tc::elect_one()) {
      uint32_t stage = 0, phase = 0;
      uint32_t pending = 0;        // stages that have been filled at least once
      uint32_t pending_phase = 0;  // parity of the phase each stage was last filled in
      bool ok = *abort_flag == 0u;
      int last_group = -1;     // expert that `landed` refers to
      uint32_t landed = 0;     // bit s: the rows of source s for that expert have landed
      for (uint32_t t = worker; t < total_tiles && ok; t += workers) {
        const TileCoord c = locate_tile<kFromStaging>(gt, num_groups, p, t, tile_m);
        if constexpr (kFromStaging) {
          // The tile's rows were stored by peers.  Wait for the arrival counters of the
          // sources it covers (rows of an expert are grouped by source rank), then order
          // the peers' (generic-proxy) stores before the TMA (async-proxy) reads.
          if (c.group != last_group) {
            last_group = c.group;
            landed = 0;
          }
          const WaitCtx w{p.status, p.timeout_ns, static_cast<uint32_t>(p.rank)};
          const uint32_t* arrived =
              reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.off_arrived_e) +
              (static_cast<size_t>(parity) * p.nle + c.group) * p.world;
          const uint32_t r0 = static_cast<uint32_t>(c.m_blk * tile_m);
          const uint32_t r1 = min(r0 + static_cast<uint32_t>(tile_m), static_cast<uint32_t>(c.rows));
          uint32_t first = 0;  // first row of source s inside the expert
          bool waited = false;
          for (int s = 0; s < p.world && ok; ++s) {
            uint32_t n;
            if (gt.src_rows != nullptr) {
              n = gt.src_rows[c.group * p.world + s];
            } else {
              // No per-source table: counts straight from the posted histograms.
              const uint32_t v = ptx::ld_relaxed_sys(
                  reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.off_counts_all) +
                  (static_cast<size_t>(parity) * p.world + s) * p.num_experts + p.rank * p.nle +
                  c.group);
              n = v > 1u ? v - 1u : 0u;
            }
            const bool overlaps = n > 0 && first < r1 && first + n > r0;
            if (overlaps && !((landed >> s) & 1u)) {
              uint32_t seen;
              ok = wait_until(arrived + s, PredGe{n}, seen, w, kPhaseFusedGemm,
                              static_cast<uint32_t>(s), n);
              landed |= 1u << s;
              waited = true;
            }
            first += n;
          }
          if (!ok) {
            *abort_flag = 1u;
            break;
          }
          if (waited) ptx::fence_proxy_async();
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = tc::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag, kWaitLimitNs);
          if (!ok) break;
          uint8_t* a_dst = stages + stage * kStageStride;
          uint8_t* b_dst = a_dst + kABytes;
          pending |= 1u << stage;
          pending_phase = (pending_phase & ~(1u << stage)) | (phase << stage);
          const int a_row = c.a_row0 + c.m_blk * tile_m + static_cast<int>(cta_rank) * kBlockM;
          if constexpr (kTwoCta) {
            // This CTA's rows of A and its half of the weight tile; the bytes of both CTAs
            // are counted on the leader's barrier, which only the leader arms.
            if (leader) tc::mbar_arrive_expect_tx(&ctl->full[stage], stage_tx_bytes);
            int b_row;
            if constexpr (SWIGLU) b_row = (cta_rank == 0 ? 0 : g.n_out) + c.n_blk * half_n;
            else b_row = c.n_blk * tile_n + static_cast<int>(cta_rank) * half_n;
            tc::tma_load_3d_2cta(a_dst, &tmap_a, &ctl->full[stage], kb * kBlockK, a_row, c.a_plane);
            tc::tma_load_3d_2cta(b_dst, &tmap_b, &ctl->full[stage], kb * kBlockK, b_row, c.w_plane);
          } else {
            tc::mbar_arrive_expect_tx(&ctl->full[stage], stage_tx_bytes);
            tc::tma_load_3d(a_dst, &tmap_a, &ctl->full[stage], kb * kBlockK, a_row, c.a_plane);
            if constexpr (SWIGLU) {
              const int row = c.n_blk * half_n;
              tc::tma_load_3d(b_dst, &tmap_b, &ctl->full[stage], kb * kBlockK, row, c.w_plane);
              tc::tma_load_3d(b_dst + b_half_bytes, &tmap_b, &ctl->full[stage], kb * kBlockK,
                              g.n_out + row, c.w_plane);
            } else {
              const int row = c.n_blk * tile_n;
              tc::tma_load_3d(b_dst, &tmap_b, &ctl->full[stage], kb * kBlockK, row, c.w_plane);
              tc::tma_load_3d(b_dst + b_half_bytes, &tmap_b, &ctl->full[stage], kb * kBlockK,
                              row + half_n, c.w_plane);
            }
          }
          if (++stage == kNumStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag != 0u) {
        // Give the loads already issued a bounded time to land before the CTA
        // leaves: their destination is this CTA's shared memory.
        uint64_t t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (int s = 0; s < kNumStages; ++s) {
          if (!((pending >> s) & 1u)) continue;
          // (The non-leader of a pair has no barrier of its own to watch; it just sits
          // out the time limit, which is far longer than any load takes.)
          while (!leader || !tc::mbar_try_wait(&ctl->full[s], (pending_phase >> s) & 1u)) {
            uint64_t t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > 100000000ull) break;  // 100 ms in total
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (leader && tc::elect_one()) {
      const uint32_t idesc = tc::make_instr_desc(1u, tile_m, tile_n);
      uint32_t stage = 0, phase = 0;
      uint32_t local = 0;
      bool ok = *abort_flag == 0u;
      for (uint32_t t = worker; t < total_tiles && ok; t += workers, ++local) {
        const uint32_t buf = local & 1u;
        const uint32_t use = local >> 1;  // how often this accumulator was used before
        ok = tc::mbar_wait(&ctl->tmem_empty[buf], (use & 1u) ^ 1u, abort_flag, kWaitLimitNs);
        if (!ok) break;
        tc::tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * kBlockN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = tc::mbar_wait(&ctl->full[stage], phase, abort_flag, kWaitLimitNs);
          if (!ok) break;
          tc::tc_fence_after_sync();
          const uint8_t* a_src = stages + stage * kStageStride;
          const uint64_t a_desc = tc::make_smem_desc_sw128(a_src);
          const uint64_t b_desc = tc::make_smem_desc_sw128(a_src + kABytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            if constexpr (kTwoCta) {
              tc::mma_f16_ss_2cta(tmem_d, tc::advance_smem_desc(a_desc, k * kUmmaK * 2),
                                  tc::advance_smem_desc(b_desc, k * kUmmaK * 2), idesc,
                                  (kb | k) != 0);
            } else {
              tc::mma_f16_ss(tmem_d, tc::advance_smem_desc(a_desc, k * kUmmaK * 2),
                             tc::advance_smem_desc(b_desc, k * kUmmaK * 2), idesc,
                             (kb | k) != 0);
            }
          }
          // Stage reusable (in both CTAs of a pair) once these MMAs have read it.
          if constexpr (kTwoCta) tc::mma_commit_2cta(&ctl->empty[stage], 0x3);
          else tc::mma_commit(&ctl->empty[stage]);
          if (++stage == kNumStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          if constexpr (kTwoCta) tc::mma_commit_2cta(&ctl->tmem_full[buf], 0x3);
          else tc::mma_commit(&ctl->tmem_full[buf]);
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    const int ew = warp - 4;  // lanes [32 * ew, 32 * ew + 32) of tensor memory
    uint32_t local = 0;
    bool ok = *abort_flag == 0u;
    const int row_bytes_out = g.n_out * 2;
    for (uint32_t t = worker; t < total_tiles && ok; t += workers, ++local) {
      const TileCoord c = locate_tile<kFromStaging>(gt, num_groups, p, t, tile_m);
      const uint32_t buf = local & 1u;
      const uint32_t use = local >> 1;
      ok = tc::mbar_wait(&ctl->tmem_full[buf], use & 1u, abort_flag, kWaitLimitNs);
      if (!ok) break;
      tc::tc_fence_after_sync();
      const int tile_row = ew * 32 + lane;
      const int row = c.m_blk * tile_m + static_cast<int>(cta_rank) * kBlockM + tile_row;
      const bool row_ok = row < c.rows;
      const int out_row = c.out_row0 + row;

      // Where this thread's row goes.
      __nv_bfloat16* local_row = nullptr;
      size_t peer_off = 0;
      const int replicas = kToPeers ? min(p.dp_size, 8) : 0;
      uint32_t sig_token = kNoSignal, sig_group = 0;
      if constexpr (kToPeers) {
        if (row_ok) {
          const uint2 rs = p.row_src[static_cast<size_t>(c.w_plane) * p.cap + out_row];
          const int src_rank = static_cast<int>(rs.x & 0xffffu);
          const uint32_t k = rs.x >> 16;
          const uint32_t token = rs.y;
          if (token < static_cast<uint32_t>(p.max_tokens) && k < static_cast<uint32_t>(p.topk) &&
              src_rank < p.world) {
            sig_token = token;
            sig_group = static_cast<uint32_t>((src_rank / p.dp_size) * p.dp_size);
            peer_off = p.off_comb_stage + (static_cast<size_t>(token) * p.topk + k) * row_bytes_out;
          } else if (p.debug_checks) {
            report_failure(p.status, kBadToken, kPhaseCombinePayload, src_rank, p.max_tokens,
                           token, p.rank);
          }
        }
      } else {
        local_row = g.out + static_cast<int64_t>(c.w_plane) * g.out_stride_e +
                    static_cast<int64_t>(out_row) * g.out_stride_row;
      }
      if constexpr (kFromStaging) {
        // First column block of a row also records where the row came from.
        if (row_ok && c.n_blk == 0) {
          const uint8_t* slot = p.peer[p.rank] + p.off_disp_stage +
                                static_cast<size_t>(c.a_row0 + row) * p.slot_bytes;
          const int4 tr = ptx::ld_cg_v4(slot + p.trailer_off);
          uint2 rs;
          rs.x = (static_cast<uint32_t>(tr.w) & 0xffffu) | (static_cast<uint32_t>(tr.y) << 16);
          rs.y = static_cast<uint32_t>(tr.x);
          p.row_src[static_cast<size_t>(c.w_plane) * p.cap + out_row] = rs;
        }
      }

      if constexpr (kToPeers) {
        // The rows' destinations, for the lanes that will store other rows' segments and for
        // the signalling below.  (Double buffered by accumulator; the barrier at the end of
        // every tile keeps the epilogue warps within one tile of each other.)
        ctl->sig_token[buf][tile_row] = sig_token;
        ctl->sig_group[buf][tile_row] = sig_group;
        peer_stage->row_off[buf][tile_row] = peer_off;
        __syncwarp();
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + buf * kBlockN;
      const int col0 = c.n_blk * out_cols_per_tile;
#pragma unroll 1
      for (int chunk = 0; chunk * 32 < out_cols_per_tile; ++chunk) {
        uint32_t acc[32];
        uint32_t packed[16];
        tc::tmem_ld_32x32(taddr + chunk * 32, acc);
        if constexpr (SWIGLU) {
          uint32_t up[32];
          tc::tmem_ld_32x32(taddr + half_n + chunk * 32, up);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g0 = __uint_as_float(acc[2 * j]), g1 = __uint_as_float(acc[2 * j + 1]);
            const float u0 = __uint_as_float(up[2 * j]), u1 = __uint_as_float(up[2 * j + 1]);
            packed[j] = pack_bf16(silu(g0) * u0, silu(g1) * u1);
          }
        } else {
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            packed[j] = pack_bf16(__uint_as_float(acc[2 * j]), __uint_as_float(acc[2 * j + 1]));
          }
        }
        const int col = col0 + chunk * 32;
        if constexpr (kToPeers) {
          uint8_t* stg = &peer_stage->rows[ew][0][0];
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            int4 q;
            q.x = packed[4 * v];
            q.y = packed[4 * v + 1];
            q.z = packed[4 * v + 2];
            q.w = packed[4 * v + 3];
            *reinterpret_cast<int4*>(stg + lane * kOutStageRowBytes + (chunk & 1) * 64 + v * 16) = q;
          }
          const bool last_chunk = (chunk + 1) * 32 >= out_cols_per_tile;
          if ((chunk & 1) == 1 || last_chunk) {
            __syncwarp();
            const int pair0 = (chunk & ~1) * 32;  // first tile column of the staged pair
            const int seg = lane & 7;             // 16-byte piece of the row's 128 bytes
            const int tcol = pair0 + seg * 8;
            const bool seg_ok = seg * 8 < ((chunk & 1) + 1) * 32 && tcol + 8 <= out_cols_per_tile &&
                                col0 + tcol + 8 <= g.n_out;
#pragma unroll 2
            for (int it = 0; it < 8; ++it) {
              const int rr = it * 4 + (lane >> 3);
              const int trow = ew * 32 + rr;
              if (seg_ok && ctl->sig_token[buf][trow] != kNoSignal) {
                const int4 q = *reinterpret_cast<const int4*>(stg + rr * kOutStageRowBytes + seg * 16);
                const uint32_t grp = ctl->sig_group[buf][trow];
                const size_t off = peer_stage->row_off[buf][trow] + static_cast<size_t>(col0 + tcol) * 2;
                for (int r = 0; r < replicas; ++r) ptx::st_v4(p.peer[grp + r] + off, q);
              }
            }
            __syncwarp();
          }
        } else {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (chunk * 32 + v * 8 + 8 > out_cols_per_tile || col + v * 8 + 8 > g.n_out) continue;
            int4 q;
            q.x = packed[4 * v];
            q.y = packed[4 * v + 1];
            q.z = packed[4 * v + 2];
            q.w = packed[4 * v + 3];
            if (row_ok) *reinterpret_cast<int4*>(local_row + col + v * 8) = q;
          }
        }
      }
      // Accumulator drained: hand it back to the MMA warp.
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kTwoCta) tc::mbar_arrive_on_leader(&ctl->tmem_empty[buf]);
        else tc::mbar_arrive(&ctl->tmem_empty[buf]);
      }

      if constexpr (kToPeers) {
        // One fence for the whole tile, then the adds.
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ew == 0) {
          ptx::fence_acq_rel_sys();
          // Arrival is counted in columns: this tile's share of the row.
          const uint32_t units = static_cast<uint32_t>(min(out_cols_per_tile, g.n_out - col0));
          for (int j = lane; j < kBlockM; j += 32) {
            const uint32_t tok = ctl->sig_token[buf][j];
            if (tok == kNoSignal) continue;
            const uint32_t grp = ctl->sig_group[buf][j];
            for (int r = 0; r < min(p.dp_size, 8); ++r) {
              ptx::red_add_relaxed_sys(
                  reinterpret_cast<uint32_t*>(p.peer[grp + r] + p.off_comb_arrived) + tok, units);
            }
          }
        }
      }
    }
  }

  // ---- teardown -------------------------------------------------------------
  tc::tc_fence_before_sync();
  __syncthreads();
  // Neither CTA of a pair may leave while the other can still touch its shared or
  // tensor memory.
  if constexpr (kTwoCta) tc::cluster_sync();
  if (warp == 2) {
    tc::tc_fence_after_sync();
    if constexpr (kTwoCta) tc::tmem_dealloc_2cta(tmem_base, kTmemCols);
    else tc::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0 && ctl->abort_flag != 0u && g.status != nullptr) *g.status = 1u;
  (void)parity;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
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

// [experts, rows, k] bf16 with k contiguous; tiles of 64 x 128 x 1, 128-byte swizzle,
// out-of-range elements read as zero.
CUtensorMap make_operand_map(const void* base, int64_t experts, int64_t rows, int64_t k,
                             int64_t stride_row_elems, int64_t stride_expert_elems,
                             int box_rows = 128) {
  PPLX_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0, "operand base must be 16-byte aligned");
  PPLX_CHECK((stride_row_elems * 2) % 16 == 0 && (stride_expert_elems * 2) % 16 == 0,
             "operand strides must be multiples of 16 bytes (8 bf16 elements)");
  CUtensorMap map;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(experts)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(stride_row_elems) * 2,
                                 static_cast<cuuint64_t>(stride_expert_elems) * 2};
  const cuuint32_t box[3] = {kBlockK, static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = encode_tiled()(
      &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PPLX_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code " << static_cast<int>(r));
  return map;
}

// `src_entries`: entries of the per-source row table of the staging-fed form (0: none);
// `to_peers`: room for the peer-storing epilogue's staging.
size_t smem_bytes(int num_groups, size_t src_entries = 0, bool to_peers = false) {
  static_assert(kStages * kStageBytes == kStages2 * kStageBytes2, "both rings use 192 KiB");
  return 1024 + kStages * kStageBytes + sizeof(SharedControl) +
         sizeof(uint32_t) * (4 * static_cast<size_t>(num_groups) + 1 + src_entries) +
         (to_peers ? sizeof(PeerStage) + 16 : 0);
}

// The per-source table is kept in shared memory when it is at most this many entries.
constexpr size_t kMaxSrcEntries = 2048;

template <bool SWIGLU, bool kFromStaging, bool kToPeers, bool kTwoCta>
void launch_one(const CUtensorMap& tmap_a, const WeightMaps& tmap_b, const GroupedGemmArgs& g,
                int num_groups, int grid, cudaStream_t stream) {
  auto* kernel = grouped_gemm_kernel<SWIGLU, kFromStaging, kToPeers, kTwoCta>;
  const size_t src_entries =
      (kFromStaging && g.src_table != 0) ? static_cast<size_t>(num_groups) * g.a2a.world : 0;
  const size_t smem = smem_bytes(num_groups, src_entries, kToPeers);
  PPLX_CHECK(smem <= 227 * 1024, "the tile tables of " << num_groups << " experts need " << smem
                                                       << " bytes of shared memory");
  CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(kTwoCta ? (grid & ~1) : grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = kTwoCta ? 2 : 1;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, tmap_a, tmap_b, g));
}

template <bool SWIGLU, bool kFromStaging, bool kToPeers>
void launch_variant(const CUtensorMap& tmap_a, const WeightMaps& tmap_b,
                    const GroupedGemmArgs& g, int num_groups, int grid, bool two_cta,
                    cudaStream_t stream) {
  if (two_cta && grid >= 2) {
    launch_one<SWIGLU, kFromStaging, kToPeers, true>(tmap_a, tmap_b, g, num_groups, grid, stream);
  } else {
    launch_one<SWIGLU, kFromStaging, kToPeers, false>(tmap_a, tmap_b, g, num_groups, grid, stream);
  }
}

// A CTA pair is ~15 % faster per flop, but an expert's last 256-row tile wastes up
// to 256 rows of MMA work (128 for single CTAs).  With rows per expert only known
// on the device, the pair form is chosen when that worst case stays small.
bool want_two_cta(const GroupedGemmCall& c) {
  if (c.cta_pair >= 0) return c.cta_pair != 0;
  const int64_t rows = c.expected_total_rows > 0
                           ? c.expected_total_rows
                           : static_cast<int64_t>(c.num_experts) * c.rows_per_expert;
  return rows / std::max(1, c.num_experts) >= 2048;
}

void check_common(const GroupedGemmCall& c) {
  PPLX_CHECK(c.num_experts > 0 && c.num_experts <= kMaxExperts, "num_experts out of range");
  PPLX_CHECK(c.k > 0 && c.k % 8 == 0, "K must be a positive multiple of 8");
  PPLX_CHECK(c.n_out > 0 && c.n_out % 8 == 0, "the output width must be a positive multiple of 8");
  PPLX_CHECK(c.half_n == 0 || (c.half_n % 8 == 0 && c.half_n >= 16 && c.half_n <= 128),
             "half_n must be a multiple of 8 in [16, 128]");
}

GroupedGemmArgs base_args(const GroupedGemmCall& c) {
  GroupedGemmArgs g{};
  g.counts = c.counts;
  g.out = static_cast<__nv_bfloat16*>(c.out);
  g.out_stride_e = c.out_stride_e;
  g.out_stride_row = c.out_stride_row;
  g.status = c.status;
  g.num_experts = c.num_experts;
  g.rows_per_expert = c.rows_per_expert;
  g.n_out = c.n_out;
  g.k = c.k;
  return g;
}

// Candidate tile widths (weight rows per B half) and one weight map for each.  A
// forced width leaves a single candidate; `units` > 0 (peer-storing epilogue) keeps
// only the widths whose column-block count divides the arrival units of a row.
WeightMaps weight_maps(const GroupedGemmCall& c, GroupedGemmArgs& g, int units) {
  static const int kCandidates[kNumTileWidths] = {128, 112, 96, 80, 64};
  const int64_t w_rows = c.swiglu ? 2 * static_cast<int64_t>(c.n_out) : c.n_out;
  WeightMaps maps{};
  int valid = 0;
  for (int i = 0; i < kNumTileWidths; ++i) {
    int half = kCandidates[i];
    if (c.half_n > 0) half = (i == 0) ? c.half_n : 0;
    if (half > 0 && units > 0 && units % ceil_div(c.n_out, 2 * half) != 0) half = 0;
    g.widths[i] = half;
    // Unused slots still need a well-formed map.
    maps.m[i] = make_operand_map(c.w, c.num_experts, w_rows, c.k, c.w_stride_row, c.w_stride_e,
                                 half > 0 ? half : 128);
    valid += half > 0;
  }
  PPLX_CHECK(valid > 0, "no tile width fits: the arrival units of a row ("
                            << units << ") must be a multiple of the output's column blocks");
  return maps;
}

}  // namespace

void launch_grouped_gemm(const GroupedGemmCall& c, cudaStream_t stream) {
  check_common(c);
  PPLX_CHECK(reinterpret_cast<uintptr_t>(c.out) % 16 == 0 && c.out_stride_row % 8 == 0 &&
                 c.out_stride_e % 8 == 0,
             "the output must be 16-byte aligned");
  const CUtensorMap tmap_a = make_operand_map(c.x, c.num_experts, c.rows_per_expert, c.k,
                                              c.x_stride_row, c.x_stride_e);
  const int grid = c.num_sms > 0 ? c.num_sms : get_sm_count();
  const bool two_cta = want_two_cta(c);
  GroupedGemmArgs g = base_args(c);
  const WeightMaps tmap_b = weight_maps(c, g, 0);
  if (c.swiglu) launch_variant<true, false, false>(tmap_a, tmap_b, g, c.num_experts, grid, two_cta, stream);
  else launch_variant<false, false, false>(tmap_a, tmap_b, g, c.num_experts, grid, two_cta, stream);
}

void launch_gemm_from_staging(const GroupedGemmCall& c, const A2AParams& p,
                              int32_t* out_num_tokens, cudaStream_t stream) {
  check_common(c);
  PPLX_CHECK(c.swiglu, "the staging-fed GEMM is the SwiGLU up projection");
  PPLX_CHECK(p.scale_bytes == 0 && p.hidden_bytes == p.hidden_dim * 2,
             "the staging-fed GEMM needs a bf16 dispatch payload without scales");
  PPLX_CHECK(c.k == p.hidden_dim && c.num_experts == p.nle && c.rows_per_expert >= p.cap,
             "shape mismatch between the GEMM and the all-to-all");
  PPLX_CHECK(reinterpret_cast<uintptr_t>(c.out) % 16 == 0 && c.out_stride_row % 8 == 0 &&
                 c.out_stride_e % 8 == 0,
             "the output must be 16-byte aligned");
  // A: [1][world * region_slots][hidden] bf16 view of this rank's packed staging.
  const int64_t slots = static_cast<int64_t>(p.world) * p.region_slots;
  const CUtensorMap tmap_a = make_operand_map(p.peer[p.rank] + p.off_disp_stage, 1, slots,
                                              p.hidden_dim, p.slot_bytes / 2,
                                              slots * p.slot_bytes / 2);
  const int grid = c.num_sms > 0 ? c.num_sms : get_sm_count();
  const bool two_cta = want_two_cta(c);
  GroupedGemmArgs g = base_args(c);
  const WeightMaps tmap_b = weight_maps(c, g, 0);
  g.out_num_tokens = out_num_tokens;
  g.a2a = p;
  g.src_table = static_cast<size_t>(p.nle) * p.world <= kMaxSrcEntries ? 1 : 0;
  launch_variant<true, true, false>(tmap_a, tmap_b, g, p.nle, grid, two_cta, stream);
}

void launch_gemm_to_peers(const GroupedGemmCall& c, const A2AParams& p, cudaStream_t stream) {
  check_common(c);
  PPLX_CHECK(!c.swiglu, "the peer-storing GEMM is the plain down projection");
  PPLX_CHECK(c.n_out == p.hidden_dim && c.num_experts == p.nle && c.rows_per_expert >= p.cap,
             "shape mismatch between the GEMM and the all-to-all");
  PPLX_CHECK(c.counts == reinterpret_cast<const int32_t*>(p.recv_count),
             "counts must be the all-to-all's received-row counts");
  const int grid = c.num_sms > 0 ? c.num_sms : get_sm_count();
  const bool two_cta = want_two_cta(c);
  PPLX_CHECK(p.dp_size <= 8, "at most 8 replicas per DP group");
  const CUtensorMap tmap_a = make_operand_map(c.x, c.num_experts, c.rows_per_expert, c.k,
                                              c.x_stride_row, c.x_stride_e);
  GroupedGemmArgs g = base_args(c);
  const WeightMaps tmap_b = weight_maps(c, g, 0);
  g.out = nullptr;
  g.a2a = p;
  launch_variant<false, false, true>(tmap_a, tmap_b, g, c.num_experts, grid, two_cta, stream);
}

}  // namespace pplx
