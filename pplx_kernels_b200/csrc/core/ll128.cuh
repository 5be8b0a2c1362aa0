// Flag-in-data transfer lines: payload that carries its own arrival flag.
//
// A row travels as 128-byte lines, each holding 120 bytes of payload followed by
// an 8-byte flag.  Eight consecutive lanes of a warp write one line with a single
// 16-byte-per-lane store instruction (lane 7 of the group holds the last 8 payload
// bytes and the flag), and the receiver reads it back the same way.  NVLink
// delivers such a store as one 128-byte write and the L2 serves the 128-byte read
// as one request, so a reader sees either the whole old line or the whole new
// one: once the flag matches, the other 120 bytes are the ones sent with it.
// (This is the property NCCL's LL128 protocol relies on for NVLink peers.)
//
// What this buys over "stores, fence, counter": the sender never waits for its
// stores to be acknowledged (no fence.sys, no red.release round trip), there is
// no separate counter hop, and the receiver can consume a row while later rows
// are still in flight.  The price is 6.7 % more bytes on the wire and 8-byte
// (instead of 16-byte) accesses on the local side of the copy.
//
// The flag is a tag plus the iteration number of the object, so a stale line of
// an earlier iteration never matches; staging memory starts zeroed and is only
// ever written in this format, so nothing else can match either.  The reference
// has no counterpart: its intranode kernels signal with a release store after a
// grid-wide barrier (intranode_dispatch.cu:184-193) and a per-token atomic
// (intranode_combine.cu:114-117).
#pragma once

#include <cstdint>

#include "ll128_layout.h"
#include "ptx.cuh"
#include "wait.cuh"

namespace pplx {
namespace ll {

constexpr uint64_t kDispatchTag = 0xD15Bull << 48;
constexpr uint64_t kCombineTag = 0xC0B1ull << 48;

__device__ __forceinline__ void st16(void* p, uint64_t a, uint64_t b) {
  asm volatile("st.volatile.global.v2.u64 [%0], {%1,%2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}

__device__ __forceinline__ void ld16(const void* p, uint64_t& a, uint64_t& b) {
  asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

// 8-byte read of an input nobody writes while the kernel runs (device or mapped host memory).
__device__ __forceinline__ uint64_t ld_src8(const void* p) {
  uint64_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u64 %0, [%1];" : "=l"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ void st8(void* p, uint64_t v) {
  asm volatile("st.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void st4(void* p, uint32_t v) {
  asm volatile("st.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded polling shared by all lanes of a warp: the first polls are free, later ones
// back off and consult the clock and the failure record through lane 0 so that the warp
// stays convergent.
struct Poll {
  const WaitCtx& w;
  uint32_t phase;
  uint32_t peer;
  uint32_t spins = 0;
  uint64_t t0 = 0;

  __device__ __forceinline__ Poll(const WaitCtx& ctx, uint32_t ph, uint32_t pr)
      : w(ctx), phase(ph), peer(pr) {}

  // Call after an unsuccessful poll (all 32 lanes).  False: give up.
  __device__ __forceinline__ bool again(int lane, uint64_t expected, uint64_t observed) {
    if (++spins < 64u) return true;
    return patient(lane, expected, observed);
  }

  // The patient part (see PPLX_COLD_PATH in wait.cuh).
  __device__ PPLX_COLD_PATH bool patient(int lane, uint64_t expected, uint64_t observed) {
    ptx::nanosleep(40);
    if ((spins & 15u) != 0u) return true;
    int go = 1;
    if (lane == 0) {
      const uint64_t now = ptx::globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (failed_already(w.status)) {
        go = 0;
      } else if (now - t0 > w.timeout_ns) {
        report_failure(w.status, kTimeout, phase, peer, static_cast<uint32_t>(expected),
                       static_cast<uint32_t>(observed), w.rank);
        go = 0;
      }
    }
    return __shfl_sync(0xffffffffu, go, 0) != 0;
  }
};

// Where the sender's copy of a row lives: global memory (device or mapped host memory,
// read through the non-coherent path) or this block's shared memory.
enum class Src { kGlobal, kShared };

template <Src S>
__device__ __forceinline__ uint64_t ld_row8(const uint8_t* p) {
  if constexpr (S == Src::kGlobal) return ld_src8(p);
  else return *reinterpret_cast<const uint64_t*>(p);
}

// Sends bytes of `src` as lines [l0, l1) of `slot`: line L carries src[L*120, L*120+120),
// zero beyond `nbytes` (a multiple of 8).  One warp, all lanes.
template <Src S = Src::kGlobal, int kBatch = 4>
__device__ __forceinline__ void warp_send_lines(uint8_t* slot, const uint8_t* src, int nbytes,
                                                int l0, int l1, uint64_t flag, int lane) {
  const int j = lane & 7, g = lane >> 3;
  for (int lb = l0; lb < l1; lb += 4 * kBatch) {
    uint64_t a[kBatch], b[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int line = lb + 4 * u + g;
      a[u] = 0;
      b[u] = 0;
      if (line < l1) {
        const int o = line * kLineData + j * 16;
        if (o + 8 <= nbytes) a[u] = ld_row8<S>(src + o);
        if (j < 7 && o + 16 <= nbytes) b[u] = ld_row8<S>(src + o + 8);
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int line = lb + 4 * u + g;
      if (line < l1) st16(slot + line * kLineBytes + j * 16, a[u], j == 7 ? flag : b[u]);
    }
  }
}

// Waits until lines [l0, l1) of `slot` carry `flag`, then copies their payload to `dst`
// (bytes beyond `nbytes` are dropped).  One warp, all lanes.  False: the wait ran out.
template <int kBatch = 4>
__device__ __forceinline__ bool warp_recv_lines(uint8_t* dst, const uint8_t* slot, int nbytes,
                                                int l0, int l1, uint64_t flag, int lane,
                                                Poll& poll) {
  const int j = lane & 7, g = lane >> 3;
  for (int lb = l0; lb < l1; lb += 4 * kBatch) {
    uint64_t a[kBatch], b[kBatch];
    while (true) {
      bool ready = true;
      uint64_t seen = flag;
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int line = lb + 4 * u + g;
        if (line < l1) {
          ld16(slot + line * kLineBytes + j * 16, a[u], b[u]);
          if (j == 7 && b[u] != flag) {
            ready = false;
            seen = b[u];
          }
        }
      }
      if (__all_sync(0xffffffffu, ready)) break;
      if (!poll.again(lane, flag, seen)) return false;
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int line = lb + 4 * u + g;
      if (line < l1) {
        const int o = line * kLineData + j * 16;
        if (o + 8 <= nbytes) st8(dst + o, a[u]);
        if (j < 7 && o + 16 <= nbytes) st8(dst + o + 8, b[u]);
      }
    }
  }
  return true;
}

// ---- word-granular lines: a short stream of 32-bit words (trailer, strided scales) ----

// Word `idx` of the meta stream of a dispatch row: 4 trailer words, then the fp32 scales.
template <Src S>
__device__ __forceinline__ uint32_t meta_word(int idx, const uint32_t (&trailer)[4],
                                              const float* scales, int64_t stride, int nscale) {
  if (idx < 4) return trailer[idx];
  if (idx - 4 < nscale) {
    const float* at = scales + static_cast<int64_t>(idx - 4) * stride;
    return __float_as_uint(S == Src::kGlobal ? __ldg(at) : *at);
  }
  return 0u;
}

template <Src S = Src::kGlobal>
__device__ __forceinline__ void warp_send_meta(uint8_t* meta, int nlines,
                                               const uint32_t (&trailer)[4], const float* scales,
                                               int64_t stride, int nscale, uint64_t flag, int lane) {
  const int j = lane & 7, g = lane >> 3;
  for (int lb = 0; lb < nlines; lb += 4) {
    const int line = lb + g;
    if (line < nlines) {
      const int w0 = (line * kLineData + j * 16) >> 2;
      const uint32_t x0 = meta_word<S>(w0, trailer, scales, stride, nscale);
      const uint32_t x1 = meta_word<S>(w0 + 1, trailer, scales, stride, nscale);
      uint64_t b = flag;
      if (j < 7) {
        const uint32_t x2 = meta_word<S>(w0 + 2, trailer, scales, stride, nscale);
        const uint32_t x3 = meta_word<S>(w0 + 3, trailer, scales, stride, nscale);
        b = static_cast<uint64_t>(x2) | (static_cast<uint64_t>(x3) << 32);
      }
      st16(meta + line * kLineBytes + j * 16,
           static_cast<uint64_t>(x0) | (static_cast<uint64_t>(x1) << 32), b);
    }
  }
}

// Receives the meta lines: scatters the scales (element stride `stride`) and returns the
// four trailer words to every lane.  False: the wait ran out.
__device__ __forceinline__ bool warp_recv_meta(const uint8_t* meta, int nlines, float* scales,
                                               int64_t stride, int nscale, uint64_t flag, int lane,
                                               Poll& poll, uint32_t (&trailer)[4]) {
  const int j = lane & 7, g = lane >> 3;
  for (int lb = 0; lb < nlines; lb += 4) {
    const int line = lb + g;
    uint64_t a = 0, b = 0;
    while (true) {
      bool ready = true;
      uint64_t seen = flag;
      if (line < nlines) {
        ld16(meta + line * kLineBytes + j * 16, a, b);
        if (j == 7 && b != flag) {
          ready = false;
          seen = b;
        }
      }
      if (__all_sync(0xffffffffu, ready)) break;
      if (!poll.again(lane, flag, seen)) return false;
    }
    if (lb == 0) {
      // Lane 0 holds line 0, words 0..3: the trailer.
      trailer[0] = __shfl_sync(0xffffffffu, static_cast<uint32_t>(a), 0);
      trailer[1] = __shfl_sync(0xffffffffu, static_cast<uint32_t>(a >> 32), 0);
      trailer[2] = __shfl_sync(0xffffffffu, static_cast<uint32_t>(b), 0);
      trailer[3] = __shfl_sync(0xffffffffu, static_cast<uint32_t>(b >> 32), 0);
    }
    if (line < nlines && nscale > 0) {
      const int w0 = (line * kLineData + j * 16) >> 2;
      const uint32_t x[4] = {static_cast<uint32_t>(a), static_cast<uint32_t>(a >> 32),
                             static_cast<uint32_t>(b), static_cast<uint32_t>(b >> 32)};
      const int nw = j < 7 ? 4 : 2;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int s = w0 + t - 4;
        if (t < nw && s >= 0 && s < nscale) scales[static_cast<int64_t>(s) * stride] = __uint_as_float(x[t]);
      }
    }
  }
  return true;
}

}  // namespace ll
}  // namespace pplx
