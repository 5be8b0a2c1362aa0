// Kernel body of grouped_gemm_fp8_sm100.cu (included there; kept in a second file
// only for length).
namespace pplx {
namespace {

struct Fp8GemmArgs {
  const int32_t* counts;   // [E]
  const float* sa;         // [E][rows][kblocks]
  int64_t sa_stride_e, sa_stride_row;
  const float* sw;         // [E][ceil(w_rows / 128)][kblocks]
  int64_t sw_stride_e, sw_stride_row;
  void* out;               // bf16 [E][rows][n_out]  or  e4m3 [E][rows][n_out]
  int64_t out_stride_e, out_stride_row;  // elements
  float* out_scale;        // kSwiGLUQuant: [E][rows][n_out / 128]
  int64_t os_stride_e, os_stride_row;
  uint32_t* status;
  int num_experts, rows_per_expert, n_out, k;
  // Only read by the forms fused with the all-to-all:
  int32_t* out_num_tokens;  // optional [nle]: per-expert totals for the caller
  int src_table;            // keep rows per (expert, source) in shared memory
  A2AParams a2a;
};

// One system-scope fence, then the queued adds on the tokens' arrival counters (one warp).
__device__ __forceinline__ void flush_signals(const A2AParams& p, const Fp8PeerStage* stage,
                                              uint32_t count, int lane) {
  ptx::fence_acq_rel_sys();
  for (uint32_t i = lane; i < count; i += 32) {
    const uint32_t tok = stage->q_token[i];
    const uint32_t grp = stage->q_group_units[i] & 0xffu;
    const uint32_t units = stage->q_group_units[i] >> 8;
    for (int r = 0; r < min(p.dp_size, 8); ++r) {
      ptx::red_add_relaxed_sys(
          reinterpret_cast<uint32_t*>(p.peer[grp + r] + p.off_comb_arrived) + tok, units);
    }
  }
  __syncwarp();
}

// kFromStaging: the A operand and its scales are read out of the dispatch staging arena
// that peers fill (packed, quantising send); tiles wait for the sources they cover.
// kToPeers: the bf16 result rows go to the combine staging of the tokens' home ranks.
// Same protocol as the bf16 kernel's forms of the same names (grouped_gemm_sm100.cu).
// Staging-fed forms: waits until the rows of tile `c` have landed, that is for the arrival
// counters of exactly the sources whose rows the tile covers.  `landed` remembers the sources
// of the current expert that were already waited for.  False: a wait ran out.
__device__ __forceinline__ bool wait_tile_sources(const A2AParams& p, const Fp8Tile& c, int parity,
                                                  const uint32_t* src_rows, uint32_t& landed) {
  const WaitCtx w{p.status, p.timeout_ns, static_cast<uint32_t>(p.rank)};
  const uint32_t* arrived = reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.off_arrived_e) +
                            (static_cast<size_t>(parity) * p.nle + c.expert) * p.world;
  const uint32_t r0 = static_cast<uint32_t>(c.m_blk * kBlockM);
  const uint32_t r1 = min(r0 + static_cast<uint32_t>(kBlockM), static_cast<uint32_t>(c.rows));
  uint32_t first = 0;
  bool waited = false, ok = true;
  for (int s = 0; s < p.world && ok; ++s) {
    uint32_t n;
    if (src_rows != nullptr) {
      n = src_rows[c.expert * p.world + s];
    } else {
      const uint32_t v = ptx::ld_relaxed_sys(
          reinterpret_cast<const uint32_t*>(p.peer[p.rank] + p.off_counts_all) +
          (static_cast<size_t>(parity) * p.world + s) * p.num_experts + p.rank * p.nle + c.expert);
      n = v > 1u ? v - 1u : 0u;
    }
    if (n > 0 && first < r1 && first + n > r0 && !((landed >> s) & 1u)) {
      uint32_t seen;
      ok = wait_until(arrived + s, PredGe{n}, seen, w, kPhaseFusedGemm, static_cast<uint32_t>(s), n);
      landed |= 1u << s;
      waited = true;
    }
    first += n;
  }
  if (ok && waited) ptx::fence_proxy_async();
  return ok;
}

// E8M0 byte of a power-of-two fp32 scale (its exponent field).
__device__ __forceinline__ uint32_t e8m0_of(float scale) {
  return (__float_as_uint(scale) >> 23) & 0xffu;
}

// The smallest power of two that is not below v (v > 0, finite).
__device__ __forceinline__ float pow2_not_below(float v) {
  const uint32_t bits = __float_as_uint(v);
  const uint32_t exp = (bits >> 23) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);
  return __uint_as_float(exp << 23);
}

template <bool kSwiGLUQuant, bool kFromStaging, bool kToPeers, bool kPow2>
__global__ void __launch_bounds__(kThreads, 1)
    grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a,
                            const __grid_constant__ CUtensorMap tmap_b,
                            const __grid_constant__ Fp8GemmArgs g) {
  static_assert(!(kFromStaging && kToPeers) && !(kToPeers && kSwiGLUQuant), "unsupported form");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* stages = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  SharedControl* ctl = reinterpret_cast<SharedControl*>(stages + kStages * kStageBytes);
  uint32_t* tile_start = reinterpret_cast<uint32_t*>(ctl + 1);  // [E + 1]
  uint32_t* rows_of = tile_start + g.num_experts + 1;             // [E] valid rows
  uint32_t* a_row0 = rows_of + g.num_experts;                     // [E] first row in the A plane
  uint32_t* src_rows =                                            // [E][world] or null
      (kFromStaging && g.src_table != 0) ? a_row0 + g.num_experts : nullptr;
  // (kToPeers only) staging of the peer-storing epilogue, behind the tables, 16-byte aligned.
  Fp8PeerStage* peer_stage = reinterpret_cast<Fp8PeerStage*>(
      (reinterpret_cast<uintptr_t>(a_row0 + g.num_experts) + 15) & ~static_cast<uintptr_t>(15));
  const A2AParams& p = g.a2a;
  int parity = 0;
  if constexpr (kFromStaging || kToPeers) parity = static_cast<int>(ptx::ld_volatile(p.iter) & 1u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  const int out_cols_per_tile = kSwiGLUQuant ? kTileN / 2 : kTileN;
  const int n_blocks = ceil_div<int>(g.n_out, out_cols_per_tile);
  const int num_kb = ceil_div<int>(g.k, kBlockKBytes);

  if (tid == 0) ctl->abort_flag = 0;
  if constexpr (kFromStaging) {
    // Role of the dispatch receive phase: rows per (source, expert) from the posted
    // histograms, the layout of the packed staging, the per-expert totals.
    for (int le = tid; le < g.num_experts; le += blockDim.x) rows_of[le] = 0;
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
      if (ok && v > 1u) atomicAdd(&rows_of[le], v - 1u);
      if (src_rows != nullptr) src_rows[le * p.world + src] = (ok && v > 1u) ? v - 1u : 0u;
    }
    __syncthreads();
    for (int le = tid; le < g.num_experts; le += blockDim.x) {
      uint32_t first = 0;
      for (int l2 = 0; l2 < le; ++l2) first += rows_of[l2];
      a_row0[le] = first;
      const uint32_t rows = min(rows_of[le], static_cast<uint32_t>(p.cap));
      tile_start[le] = static_cast<uint32_t>(ceil_div<int>(static_cast<int>(rows), kBlockM) * n_blocks);
      if (blockIdx.x == 0) {
        if (g.out_num_tokens != nullptr) g.out_num_tokens[le] = static_cast<int32_t>(rows_of[le]);
        p.recv_count[le] = rows;
      }
    }
    __syncthreads();
    for (int le = tid; le < g.num_experts; le += blockDim.x)
      rows_of[le] = min(rows_of[le], static_cast<uint32_t>(p.cap));
  } else {
    for (int e = tid; e < g.num_experts; e += blockDim.x) {
      const int rows = min(max(g.counts[e], 0), g.rows_per_expert);
      rows_of[e] = static_cast<uint32_t>(rows);
      a_row0[e] = 0;
      tile_start[e] = static_cast<uint32_t>(ceil_div<int>(rows, kBlockM) * n_blocks);
    }
  }
  if constexpr (kToPeers) {
    if (blockIdx.x == 0) {
      // Role of the combine send phase's first block: the dispatch that produced these
      // rows is over on this rank, so clear its flag set and move on.
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
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&ctl->full[s], kPow2 ? 2 : 1);  // the tiles, and (kPow2) the scales
      tc::mbar_init(&ctl->empty[s], 1);
    }
    tc::mbar_init(&ctl->acc_full, 1);
    tc::mbar_init(&ctl->acc_empty, 8);
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&ctl->part_full[b], 1);
      tc::mbar_init(&ctl->part_empty[b], 8);
    }
    tc::fence_mbar_init();
    tc::tma_prefetch_desc(&tmap_a);
    tc::tma_prefetch_desc(&tmap_b);
  }
  __syncthreads();
  if (warp == 0) warp_exclusive_scan_smem(tile_start, g.num_experts, lane, true);
  if (warp == 2) {
    tc::tmem_alloc(&ctl->tmem_base, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t total_tiles = tile_start[g.num_experts];

  if (warp == 0) {
    if (tc::elect_one()) {
      uint32_t stage = 0, phase = 0, pending = 0, pending_phase = 0;
      bool ok = *abort_flag == 0u;
      int last_group = -1;  // expert that `landed` refers to
      uint32_t landed = 0;  // bit s: the rows of source s for that expert have landed
      for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Fp8Tile c = locate(tile_start, rows_of, g.num_experts, t);
        if constexpr (kFromStaging) {
          if (c.expert != last_group) {
            last_group = c.expert;
            landed = 0;
          }
          ok = wait_tile_sources(p, c, parity, src_rows, landed);
          if (!ok) {
            *abort_flag = 1u;
            break;
          }
        }
        const int a_row = static_cast<int>(a_row0[c.expert]) + c.m_blk * kBlockM;
        const int a_plane = kFromStaging ? 0 : c.expert;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = tc::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag, kWaitLimitNs);
          if (!ok) break;
          uint8_t* a_dst = stages + stage * kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          tc::mbar_arrive_expect_tx(&ctl->full[stage], kStageBytes);
          pending |= 1u << stage;
          pending_phase = (pending_phase & ~(1u << stage)) | (phase << stage);
          tc::tma_load_3d(a_dst, &tmap_a, &ctl->full[stage], kb * kBlockKBytes, a_row, a_plane);
          // Two halves of 128 weight rows: gate and up rows, or consecutive rows.
          const int row0 = kSwiGLUQuant ? c.n_blk * (kTileN / 2) : c.n_blk * kTileN;
          const int row1 = kSwiGLUQuant ? g.n_out + row0 : row0 + kTileN / 2;
          tc::tma_load_3d(b_dst, &tmap_b, &ctl->full[stage], kb * kBlockKBytes, row0, c.expert);
          tc::tma_load_3d(b_dst + kBBytes / 2, &tmap_b, &ctl->full[stage], kb * kBlockKBytes, row1,
                          c.expert);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag != 0u) {
        const uint64_t t0 = ptx::globaltimer_ns();
        for (int s = 0; s < kStages; ++s) {
          if (!((pending >> s) & 1u)) continue;
          while (!tc::mbar_try_wait(&ctl->full[s], (pending_phase >> s) & 1u)) {
            if (ptx::globaltimer_ns() - t0 > 100000000ull) break;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (tc::elect_one()) {
      // kind::f8f6f4, e4m3 x e4m3 -> f32, M = 128, N = 256.
      const uint32_t idesc = tc::make_instr_desc(0u, kBlockM, kTileN);
      uint32_t stage = 0, phase = 0, round = 0;
      bool ok = *abort_flag == 0u;
      if constexpr (kPow2) {
        uint32_t tile_it = 0;
        for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_it) {
          // The fold warps have read the previous tile out of the accumulator.
          ok = tc::mbar_wait(&ctl->acc_empty, (tile_it & 1u) ^ 1u, abort_flag, kWaitLimitNs);
          for (int kb = 0; kb < num_kb && ok; ++kb) {
            ok = tc::mbar_wait(&ctl->full[stage], phase, abort_flag, kWaitLimitNs);
            if (!ok) break;
            tc::tc_fence_after_sync();
            const uint8_t* a_src = stages + stage * kStageBytes;
            const uint64_t a_desc = tc::make_smem_desc_sw128(a_src);
            const uint64_t b_desc = tc::make_smem_desc_sw128(a_src + kABytes);
            const uint8_t* sf = ctl->sf[stage];
            tc::tmem_cp_32x128b_warpx4(tmem_base + kSfaCol, tc::make_smem_desc_rows16(sf));
            tc::tmem_cp_32x128b_warpx4(tmem_base + kSfbCol,
                                       tc::make_smem_desc_rows16(sf + kSfAtomBytes));
            tc::tmem_cp_32x128b_warpx4(tmem_base + kSfbCol + 4,
                                       tc::make_smem_desc_rows16(sf + 2 * kSfAtomBytes));
#pragma unroll
            for (uint32_t k = 0; k < kBlockKBytes / kUmmaKBytes; ++k) {
              tc::mma_mxf8_ss(tmem_base, tc::advance_smem_desc(a_desc, k * kUmmaKBytes),
                              tc::advance_smem_desc(b_desc, k * kUmmaKBytes),
                              tc::make_instr_desc_mxf8(kBlockM, kTileN, k),
                              (tmem_base + kSfaCol) | (k << 30), (tmem_base + kSfbCol) | (k << 30),
                              kb != 0 || k != 0);
            }
            tc::mma_commit(&ctl->empty[stage]);
            if (kb == num_kb - 1) tc::mma_commit(&ctl->acc_full);
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      for (uint32_t t = blockIdx.x; !kPow2 && t < total_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < num_kb && ok; ++kb, ++round) {
          // K blocks alternate between the two scratch accumulators.
          const uint32_t buf = round & 1u;
          ok = tc::mbar_wait(&ctl->part_empty[buf], ((round >> 1) & 1u) ^ 1u, abort_flag,
                             kWaitLimitNs);
          if (!ok) break;
          ok = tc::mbar_wait(&ctl->full[stage], phase, abort_flag, kWaitLimitNs);
          if (!ok) break;
          tc::tc_fence_after_sync();
          const uint8_t* a_src = stages + stage * kStageBytes;
          const uint64_t a_desc = tc::make_smem_desc_sw128(a_src);
          const uint64_t b_desc = tc::make_smem_desc_sw128(a_src + kABytes);
#pragma unroll
          for (int k = 0; k < kBlockKBytes / kUmmaKBytes; ++k) {
            tc::mma_f8_ss(tmem_base + buf * kTileN, tc::advance_smem_desc(a_desc, k * kUmmaKBytes),
                          tc::advance_smem_desc(b_desc, k * kUmmaKBytes), idesc, k != 0);
          }
          tc::mma_commit(&ctl->empty[stage]);
          tc::mma_commit(&ctl->part_full[buf]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (kPow2 && warp == 3) {
    // The scales of each K block as E8M0 bytes, where tcgen05.cp finds them.  Lane l owns
    // rows l, l + 32, l + 64, l + 96 of the tile: exactly one 16-byte row of the A atom.
    uint32_t stage = 0, phase = 0;
    bool ok = *abort_flag == 0u;
    uint32_t not_pow2 = 0;   // mantissa bits seen in any scale: the caller's promise was broken
    int sf_group = -1;       // kFromStaging: expert that sf_landed refers to
    uint32_t sf_landed = 0;  // (lane 0) sources of that expert already waited for
    constexpr int kChunk = 8;  // K blocks whose scales are fetched together
    for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Fp8Tile c = locate(tile_start, rows_of, g.num_experts, t);
      if constexpr (kFromStaging) {
        // The scales sit behind the rows in the staging that peers write: wait for the same
        // sources as the TMA producer does (lane 0 acquires, the warp follows).
        if (c.expert != sf_group) {
          sf_group = c.expert;
          sf_landed = 0;
        }
        int good = 1;
        if (lane == 0) good = wait_tile_sources(p, c, parity, src_rows, sf_landed) ? 1 : 0;
        good = __shfl_sync(0xffffffffu, good, 0);
        __syncwarp();
        if (good == 0) {
          if (lane == 0) *abort_flag = 1u;
          ok = false;
          break;
        }
      }
      const float* sa_rows[4];
      bool live[4];
#pragma unroll
      for (int r1 = 0; r1 < 4; ++r1) {
        const int row = c.m_blk * kBlockM + lane + 32 * r1;
        live[r1] = row < c.rows;
        if constexpr (kFromStaging) {
          sa_rows[r1] = reinterpret_cast<const float*>(
              p.peer[p.rank] + p.off_disp_stage +
              (static_cast<size_t>(a_row0[c.expert]) + (live[r1] ? row : 0)) * p.slot_bytes +
              p.hidden_bytes);
        } else {
          sa_rows[r1] = g.sa + c.expert * g.sa_stride_e + (live[r1] ? row : 0) * g.sa_stride_row;
        }
      }
      const int wrow0 = kSwiGLUQuant ? c.n_blk * (kTileN / 2) : c.n_blk * kTileN;
      const int wrow1 = kSwiGLUQuant ? g.n_out + wrow0 : wrow0 + kTileN / 2;
      const int last_block = (((kSwiGLUQuant ? 2 : 1) * g.n_out) - 1) / 128;
      const float* sw0 =
          g.sw + c.expert * g.sw_stride_e + min(wrow0 / 128, last_block) * g.sw_stride_row;
      const float* sw1 =
          g.sw + c.expert * g.sw_stride_e + min(wrow1 / 128, last_block) * g.sw_stride_row;
      // Four row bytes and two column-half bytes per K block, fetched a chunk ahead of use.
      uint32_t ea[kChunk], eb[kChunk], ea_next[kChunk], eb_next[kChunk];
      auto fetch = [&](int kb0, uint32_t (&da)[kChunk], uint32_t (&db)[kChunk]) {
#pragma unroll
        for (int u = 0; u < kChunk; ++u) {
          const int kb = min(kb0 + u, num_kb - 1);
          uint32_t v = 0;
#pragma unroll
          for (int r1 = 0; r1 < 4; ++r1) {
            uint32_t byte = 127u;
            if (live[r1]) {
              const float sc = kFromStaging ? __ldcg(sa_rows[r1] + kb) : __ldg(sa_rows[r1] + kb);
              not_pow2 |= __float_as_uint(sc) & 0x7fffffu;
              byte = e8m0_of(sc);
            }
            v |= byte << (8 * r1);
          }
          da[u] = v;
          const float w0 = __ldg(sw0 + kb), w1 = __ldg(sw1 + kb);
          not_pow2 |= (__float_as_uint(w0) | __float_as_uint(w1)) & 0x7fffffu;
          db[u] = e8m0_of(w0) | (e8m0_of(w1) << 8);
        }
      };
      fetch(0, ea_next, eb_next);
      for (int kb0 = 0; kb0 < num_kb && ok; kb0 += kChunk) {
#pragma unroll
        for (int u = 0; u < kChunk; ++u) {
          ea[u] = ea_next[u];
          eb[u] = eb_next[u];
        }
        if (kb0 + kChunk < num_kb) fetch(kb0 + kChunk, ea_next, eb_next);
#pragma unroll
        for (int u = 0; u < kChunk; ++u) {
          if (kb0 + u >= num_kb || !ok) continue;
          ok = tc::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag, kWaitLimitNs);
          if (!ok) continue;
          uint8_t* sf = ctl->sf[stage];
          uint4 a;
          a.x = (ea[u] & 0xffu) * 0x01010101u;
          a.y = ((ea[u] >> 8) & 0xffu) * 0x01010101u;
          a.z = ((ea[u] >> 16) & 0xffu) * 0x01010101u;
          a.w = (ea[u] >> 24) * 0x01010101u;
          *reinterpret_cast<uint4*>(sf + 16 * lane) = a;
          const uint32_t b0 = (eb[u] & 0xffu) * 0x01010101u;
          const uint32_t b1 = (eb[u] >> 8) * 0x01010101u;
          *reinterpret_cast<uint4*>(sf + kSfAtomBytes + 16 * lane) = make_uint4(b0, b0, b0, b0);
          *reinterpret_cast<uint4*>(sf + 2 * kSfAtomBytes + 16 * lane) = make_uint4(b1, b1, b1, b1);
          ptx::fence_proxy_async_smem();  // these writes, before tcgen05.cp reads them
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&ctl->full[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    // A scale with mantissa bits would have been truncated to its exponent: report it
    // (status 2) instead of returning plausible, wrong numbers.
    if (__any_sync(0xffffffffu, not_pow2 != 0u) && lane == 0 && g.status != nullptr)
      atomicMax(g.status, 2u);
  } else if (warp >= 4) {
    const int ew = (warp - 4) & 3;      // tensor-memory lanes [32 * ew, +32)
    const int half = (warp - 4) >> 2;   // columns [64 * half, +64) of each 128-column half
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
    uint32_t round = 0;
    uint32_t tile_it = 0;          // kPow2: tiles this CTA has finished
    uint32_t pending_signals = 0;  // kToPeers, warp 4: queued arrival adds
    bool ok = *abort_flag == 0u;
    for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Fp8Tile c = locate(tile_start, rows_of, g.num_experts, t);
      const int tile_row = ew * 32 + lane;
      const int row = c.m_blk * kBlockM + tile_row;
      const bool row_ok = row < c.rows;
      const int safe_row = row_ok ? row : 0;
      const float* sa_row;
      if constexpr (kFromStaging) {
        // The row's scales sit behind its payload in the staging slot that a peer wrote.
        sa_row = reinterpret_cast<const float*>(
            p.peer[p.rank] + p.off_disp_stage +
            (static_cast<size_t>(a_row0[c.expert]) + safe_row) * p.slot_bytes + p.hidden_bytes);
      } else {
        sa_row = g.sa + c.expert * g.sa_stride_e + safe_row * g.sa_stride_row;
      }

      if constexpr (kFromStaging) {
        // The first column block of a row also records where the row came from.
        if (row_ok && c.n_blk == 0 && half == 0) {
          const uint8_t* slot = p.peer[p.rank] + p.off_disp_stage +
                                (static_cast<size_t>(a_row0[c.expert]) + row) * p.slot_bytes;
          const int4 tr = ptx::ld_cg_v4(slot + p.trailer_off);
          uint2 rs;
          rs.x = (static_cast<uint32_t>(tr.w) & 0xffffu) | (static_cast<uint32_t>(tr.y) << 16);
          rs.y = static_cast<uint32_t>(tr.x);
          p.row_src[static_cast<size_t>(c.expert) * p.cap + row] = rs;
        }
      }
      // Weight scale rows of the two halves of the tile.
      const int wrow0 = kSwiGLUQuant ? c.n_blk * (kTileN / 2) : c.n_blk * kTileN;
      const int wrow1 = kSwiGLUQuant ? g.n_out + wrow0 : wrow0 + kTileN / 2;
      const int last_block = (((kSwiGLUQuant ? 2 : 1) * g.n_out) - 1) / 128;
      const float* sw0 =
          g.sw + c.expert * g.sw_stride_e + min(wrow0 / 128, last_block) * g.sw_stride_row;
      const float* sw1 =
          g.sw + c.expert * g.sw_stride_e + min(wrow1 / 128, last_block) * g.sw_stride_row;

      // acc[0..63]: columns 64*half.. of the first 128-column half of the tile,
      // acc[64..127]: the same columns of the second half.
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      if constexpr (kPow2) {
        // The tensor cores applied the scales: take the finished tile out of tensor memory
        // and hand the accumulator back before converting and storing.
        ok = tc::mbar_wait(&ctl->acc_full, tile_it & 1u, abort_flag, kWaitLimitNs);
        ++tile_it;
        if (ok) {
          tc::tc_fence_after_sync();
          // Four loads of 32 columns in flight, one wait: the accumulator is free again
          // after a single tensor-memory round trip.
          const uint32_t t_acc = t_lane + half * 64;
          uint32_t raw[4][32];
#pragma unroll
          for (int q = 0; q < 4; ++q) tc::tmem_ld_32x32(t_acc + (q >> 1) * 128 + (q & 1) * 32, raw[q]);
          tc::tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[q * 32 + j] = __uint_as_float(raw[q][j]);
          }
          tc::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&ctl->acc_empty);
        }
      }
      for (int kb = 0; !kPow2 && kb < num_kb && ok; ++kb, ++round) {
        // Staging memory is rewritten by peers every step: read it from L2, never through
        // the non-coherent path.
        const float a_scale = kFromStaging ? __ldcg(sa_row + kb) : __ldg(sa_row + kb);
        const float s0 = a_scale * __ldg(sw0 + kb);
        const float s1 = a_scale * __ldg(sw1 + kb);
        const uint32_t buf = round & 1u;
        ok = tc::mbar_wait(&ctl->part_full[buf], (round >> 1) & 1u, abort_flag, kWaitLimitNs);
        if (!ok) break;
        tc::tc_fence_after_sync();
        const uint32_t t_part = t_lane + buf * kTileN + half * 64;
#pragma unroll
        for (int q = 0; q < 8; ++q) {  // 8 pieces of 16 columns: 4 per tile half
          uint32_t part[16];
          tmem_ld_32x16(t_part + (q >> 2) * 128 + (q & 3) * 16, part);
          tc::tmem_ld_wait();
          const float s = (q >> 2) == 0 ? s0 : s1;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            acc[q * 16 + j] = fmaf(__uint_as_float(part[j]), s, acc[q * 16 + j]);
          }
        }
        tc::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&ctl->part_empty[buf]);
      }
      // All eight epilogue warps leave together or not at all: the barriers below must
      // never be entered by only some of them.
      {
        uint32_t all_ok;
        asm volatile(
            "{\n\t"
            ".reg .pred p, q;\n\t"
            "setp.ne.u32 q, %1, 0;\n\t"
            "bar.red.and.pred p, 1, 256, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(all_ok)
            : "r"(ok ? 1u : 0u)
            : "memory");
        ok = all_ok != 0u;
      }
      if (!ok) break;

      // ---- tile epilogue ------------------------------------------------------
      if constexpr (kSwiGLUQuant) {
        // acc[0..63] = gate, acc[64..127] = up for output columns 64*half.. of this tile's
        // 128 output columns (one scale block); the row maximum needs the other half too.
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          acc[j] = silu(acc[j]) * acc[64 + j];
          amax = fmaxf(amax, fabsf(acc[j]));
        }
        ctl->row_amax[half][tile_row] = amax;
        asm volatile("bar.sync 2, 256;" ::: "memory");
        amax = fmaxf(fmaxf(ctl->row_amax[0][tile_row], ctl->row_amax[1][tile_row]), 1e-4f);
        // The scale of the row's 128 outputs: amax / 448, or the next power of two above it
        // where the consumer wants hardware scales.
        const float out_scale = kPow2 ? pow2_not_below(amax / 448.0f) : amax / 448.0f;
        const float inv = 1.0f / out_scale;
        if (row_ok) {
          const int col0 = c.n_blk * 128 + half * 64;
          uint8_t* orow = static_cast<uint8_t*>(g.out) + c.expert * g.out_stride_e +
                          static_cast<int64_t>(row) * g.out_stride_row + col0;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 16 + 16 > g.n_out) continue;
            uint32_t q[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int b = v * 16 + 4 * j;
              const uint32_t p0 = __nv_cvt_float2_to_fp8x2(
                  make_float2(acc[b] * inv, acc[b + 1] * inv), __NV_SATFINITE, __NV_E4M3);
              const uint32_t p1 = __nv_cvt_float2_to_fp8x2(
                  make_float2(acc[b + 2] * inv, acc[b + 3] * inv), __NV_SATFINITE, __NV_E4M3);
              q[j] = p0 | (p1 << 16);
            }
            int4 o;
            o.x = q[0];
            o.y = q[1];
            o.z = q[2];
            o.w = q[3];
            *reinterpret_cast<int4*>(orow + v * 16) = o;
          }
          if (half == 0) {
            g.out_scale[c.expert * g.os_stride_e + static_cast<int64_t>(row) * g.os_stride_row +
                        c.n_blk] = out_scale;
          }
        }
        // row_amax is rewritten by the next tile only after every warp passed this point.
        asm volatile("bar.sync 3, 256;" ::: "memory");
      } else {
        // Where this thread's row goes (kToPeers), and whose token it is.  Looked up only now,
          // so that the pointers are not live across the K loop.
        size_t peer_off = 0;  // offset of the row's slot in the home ranks' arenas
        const int replicas = kToPeers ? min(p.dp_size, 8) : 0;
        uint32_t sig_token = kNoSignalFp8, sig_group = 0;
        if constexpr (kToPeers) {
          if (row_ok) {
            const uint2 rs = p.row_src[static_cast<size_t>(c.expert) * p.cap + row];
            const int src_rank = static_cast<int>(rs.x & 0xffffu);
            const uint32_t k = rs.x >> 16;
            const uint32_t token = rs.y;
            if (token < static_cast<uint32_t>(p.max_tokens) && k < static_cast<uint32_t>(p.topk) &&
                src_rank < p.world) {
              sig_token = token;
              sig_group = static_cast<uint32_t>((src_rank / p.dp_size) * p.dp_size);
              peer_off = p.off_comb_stage +
                         (static_cast<size_t>(token) * p.topk + k) * (static_cast<size_t>(g.n_out) * 2);
            } else if (half == 0) {
              report_failure(p.status, kBadToken, kPhaseCombinePayload, src_rank, p.max_tokens,
                             token, p.rank);
            }
          }
        }
        if constexpr (kToPeers) {
          // A thread owns one row; stored straight from registers its 16-byte pieces would
          // cross NVLink one by one.  Each warp passes 32 columns at a time through shared
          // memory and writes them out as 64-byte row segments (four lanes per row).
          if (half == 0) {
            ctl->sig_token[tile_row] = sig_token;
            ctl->sig_group[tile_row] = sig_group;
            peer_stage->row_off[tile_row] = peer_off;
          }
          asm volatile("bar.sync 2, 256;" ::: "memory");
          uint8_t* stg = &peer_stage->rows[warp - 4][0][0];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {  // 32 columns of this thread's 128
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              const int v = q4 * 4 + v4;
              int4 o;
              uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 b =
                    __floats2bfloat162_rn(acc[v * 8 + 2 * j], acc[v * 8 + 2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&b);
              }
              *reinterpret_cast<int4*>(stg + lane * kFp8StageRowBytes + v4 * 16) = o;
            }
            __syncwarp();
            const int seg = lane & 3;
            const int col = c.n_blk * kTileN + (q4 >> 1) * 128 + half * 64 + (q4 & 1) * 32 + seg * 8;
#pragma unroll 2
            for (int it = 0; it < 4; ++it) {
              const int rr = it * 8 + (lane >> 2);
              const int trow = ew * 32 + rr;
              const uint32_t tok = ctl->sig_token[trow];
              if (tok != kNoSignalFp8 && col + 8 <= g.n_out) {
                const int4 o = *reinterpret_cast<const int4*>(stg + rr * kFp8StageRowBytes + seg * 16);
                const uint32_t grp = ctl->sig_group[trow];
                const size_t off = peer_stage->row_off[trow] + static_cast<size_t>(col) * 2;
                for (int r = 0; r < replicas; ++r) ptx::st_v4(p.peer[grp + r] + off, o);
              }
            }
            __syncwarp();
          }
        } else if (row_ok) {
          __nv_bfloat16* orow = static_cast<__nv_bfloat16*>(g.out) + c.expert * g.out_stride_e +
                                static_cast<int64_t>(row) * g.out_stride_row;
#pragma unroll
          for (int v = 0; v < 16; ++v) {  // 16 vectors of 8 columns
            const int col = c.n_blk * kTileN + (v >> 3) * 128 + half * 64 + (v & 7) * 8;
            if (col + 8 > g.n_out) continue;
            int4 o;
            uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 b =
                  __floats2bfloat162_rn(acc[v * 8 + 2 * j], acc[v * 8 + 2 * j + 1]);
              w[j] = *reinterpret_cast<const uint32_t*>(&b);
            }
            *reinterpret_cast<int4*>(orow + col) = o;
          }
        }
        if constexpr (kToPeers) {
          // One fence for the whole tile, then the adds on the tokens' arrival counters.
          // (All eight warps meet at the barrier at the top of the next tile's epilogue
          // before anyone rewrites the sig arrays.)
          asm volatile("bar.sync 3, 256;" ::: "memory");
          if (warp == 4) {
            // Arrival is counted in columns: this tile's share of the row.  The adds are
            // queued and flushed behind ONE system-scope fence for as many tiles as the queue
            // holds: with a handful of rows per expert (decode) a fence per tile would cost
            // more than the tile.
            const uint32_t units =
                static_cast<uint32_t>(min(kTileN, g.n_out - c.n_blk * kTileN));
            if (pending_signals + kBlockM > kSignalQueue) {
              flush_signals(p, peer_stage, pending_signals, lane);
              pending_signals = 0;
            }
            for (int j0 = 0; j0 < kBlockM; j0 += 32) {
              const int j = j0 + lane;
              const uint32_t tok = ctl->sig_token[j];
              const bool live = tok != kNoSignalFp8;
              const uint32_t mask = __ballot_sync(0xffffffffu, live);
              if (live) {
                const uint32_t at = pending_signals + __popc(mask & ((1u << lane) - 1u));
                peer_stage->q_token[at] = tok;
                peer_stage->q_group_units[at] = ctl->sig_group[j] | (units << 8);
              }
              pending_signals += __popc(mask);
            }
          }
        }
      }
    }
    if constexpr (kToPeers) {
      // What is still queued (also after a failed wait: rows that were stored are announced).
      if (warp == 4 && pending_signals > 0) flush_signals(p, peer_stage, pending_signals, lane);
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0 && ctl->abort_flag != 0u && g.status != nullptr) atomicMax(g.status, 1u);
  (void)parity;
}

}  // namespace
}  // namespace pplx
