// Host side of the dispatch/combine all-to-all.
//
// Role parity: `SplitMode` + `AllToAll` (csrc/all_to_all/all_to_all.h:9-71),
// `AllToAllIntraNode` (intranode.h:21-89) and `AllToAllInterNode`
// (internode.h:16-133).  One class serves both API flavours: inside one NVSwitch
// box every peer is reachable by load/store, so "internode" differs only in how
// the ranks find one another.  Relaxations against the reference: a single DP
// group (including world_size 1) is accepted.  num_experts need not divide evenly over
// the ranks: each rank owns ceil(num_experts / world_size) expert slots and the last
// rank(s) fewer real experts (the reference mixes ceil and floor there).
#pragma once

#include <memory>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "../core/buffer.h"
#include "../core/ll128_layout.h"
#include "../core/status.h"
#include "../kernels/a2a_kernels.h"
#include "../kernels/a2a_params.h"
#include "symm_heap.h"

namespace pplx {

enum class SplitMode { kNone = 0, kSend = 1, kRecv = 2 };

inline SplitMode split_mode(bool do_send, bool do_recv) {
  if (do_send && do_recv) return SplitMode::kNone;
  if (do_send) return SplitMode::kSend;
  if (do_recv) return SplitMode::kRecv;
  throw Error("dispatch/combine called with do_send = do_recv = false");
}

// Human-readable rendering of a failure record.
std::string describe_status(const Status& s);

struct A2AConfig {
  int max_num_tokens = 0;
  int num_experts = 0;
  int experts_per_token = 0;
  int rank = 0;
  int world_size = 1;
  int dp_size = 1;
  int hidden_dim = 0;
  int hidden_dim_bytes = 0;
  int hidden_dim_scale_bytes = 0;
};

// Tensor arguments of one dispatch call (everything except the object itself).
struct DispatchCall {
  int32_t* out_num_tokens = nullptr;
  Strided3D<uint8_t> out_x;   // strides in bytes; stride_col unused
  Strided3D<float> out_scale; // optional (data == nullptr), strides in elements
  Strided2D<const uint8_t> x; // row stride in bytes
  Strided2D<const float> x_scale;
  const uint32_t* indices = nullptr;
  const uint32_t* bound_m = nullptr;
  int num_tokens = 0;
  // Capacity checks (rows per expert the caller's buffers can hold).
  int64_t out_rows = 0;
  // x holds bf16 values (hidden_dim_bytes of them per row) that the send quantises to
  // e4m3 + fp32 scale per 128 columns; x_scale is then unused.
  bool quantize = false;
  // x, x_scale and indices are device aliases of mapped pinned host memory: the send reads
  // the tokens across PCIe itself and no upload precedes the call.
  bool x_on_host = false;
};

struct CombineCall {
  void* out_tokens = nullptr;
  int64_t out_stride_row = 0;  // elements
  const float* weights = nullptr;
  int64_t w_stride_row = 0;
  const void* expert_y = nullptr;
  int64_t y_stride_e = 0;      // elements
  int64_t y_stride_row = 0;
  const uint32_t* bound_m = nullptr;
  int num_tokens = 0;
  DType in = DType::kBF16;
  DType out = DType::kBF16;
};

// Weights and intermediate buffer of the fused expert FFN (bf16, strides in elements).
struct FusedFfnCall {
  const void* w = nullptr;   // up: [nle][2 * inter][hidden]; down: [nle][hidden][inter]
  int64_t w_stride_e = 0;
  int64_t w_stride_row = 0;
  void* h = nullptr;         // [nle][rows_per_expert][inter]: written by up, read by down
  int64_t h_stride_e = 0;
  int64_t h_stride_row = 0;
  int rows_per_expert = 0;
  int inter_dim = 0;
  int32_t* out_num_tokens = nullptr;  // up only, optional
  uint32_t* status = nullptr;         // optional device word, 1 if a pipeline wait ran out
  int64_t expected_total_rows = 0;    // hint for the tile shape choice, 0 = capacity
};

// The same for the block-scaled fp8 layer: e4m3 weights with one fp32 scale per 128 x 128
// block, an e4m3 intermediate with one fp32 scale per row and 128 columns.  Payload strides
// in bytes (= elements), scale strides in floats.
struct FusedFfnFp8Call {
  const void* w = nullptr;    // up: [nle][2 * inter][hidden]; down: [nle][hidden][inter]
  int64_t w_stride_e = 0, w_stride_row = 0;
  const float* sw = nullptr;  // [nle][ceil(w rows / 128)][ceil(k / 128)]
  int64_t sw_stride_e = 0, sw_stride_row = 0;
  void* h = nullptr;          // e4m3 [nle][rows_per_expert][inter]: written by up, read by down
  int64_t h_stride_e = 0, h_stride_row = 0;
  float* h_scale = nullptr;   // [nle][rows_per_expert][inter / 128]
  int64_t hs_stride_e = 0, hs_stride_row = 0;
  int rows_per_expert = 0;
  int inter_dim = 0;
  int32_t* out_num_tokens = nullptr;  // up only, optional
  uint32_t* status = nullptr;
};

class AllToAll {
 public:
  AllToAll(const A2AConfig& cfg, std::shared_ptr<SymmetricAllocation> arena);
  ~AllToAll();
  AllToAll(const AllToAll&) = delete;
  AllToAll& operator=(const AllToAll&) = delete;

  // Bytes of symmetric memory one rank needs for `cfg`.
  static size_t arena_bytes(const A2AConfig& cfg);
  static void validate(const A2AConfig& cfg);

  // Collective: allocates the arena through `bs` and builds the object.
  static std::unique_ptr<AllToAll> create(const A2AConfig& cfg, Bootstrap& bs);

  // `cfg.world_size` ranks on the current device; cfg.rank is ignored.
  static std::vector<std::unique_ptr<AllToAll>> create_local_world(const A2AConfig& cfg);

  void dispatch(const DispatchCall& call, SplitMode mode, cudaStream_t stream);
  void combine(const CombineCall& call, SplitMode mode, cudaStream_t stream);

  // Send half of the two-hop "packed" dispatch: rows land in the destination's staging
  // grouped by local expert, ready for fused_up.  The payload is bf16 without scales, or
  // (call.quantize, on an object created for a 1-byte payload with scales) bf16 tokens
  // converted to e4m3 + one fp32 scale per 128 columns on the way.  Only x, indices,
  // bound_m, num_tokens and quantize of the call are used.
  void dispatch_send_packed(const DispatchCall& call, cudaStream_t stream);
  static void dispatch_send_packed_group(const std::vector<AllToAll*>& ranks,
                                         const std::vector<DispatchCall>& calls,
                                         cudaStream_t stream);
  DispatchArgs make_packed_send_args(const DispatchCall& call) const;

  // Fused MoE path: dispatch_send_packed, fused_up, fused_down, combine(kRecv).
  // fused_up takes the place of the dispatch receive phase (the tcgen05 GEMM reads
  // the staging arena as peers fill it), fused_down that of the combine send phase
  // (the GEMM epilogue stores to the tokens' home ranks).
  void fused_up(const FusedFfnCall& call, cudaStream_t stream);
  void fused_down(const FusedFfnCall& call, cudaStream_t stream);
  // fp8 forms: after dispatch_send_packed with call.quantize (bf16 tokens quantised to e4m3
  // + fp32 scale per 128 columns while they are sent).
  void fused_up_fp8(const FusedFfnFp8Call& call, cudaStream_t stream);
  void fused_down_fp8(const FusedFfnFp8Call& call, cudaStream_t stream);

  // All ranks of a local world in one cooperative launch per operation.
  static void dispatch_group(const std::vector<AllToAll*>& ranks,
                             const std::vector<DispatchCall>& calls, SplitMode mode,
                             cudaStream_t stream);
  static void combine_group(const std::vector<AllToAll*>& ranks,
                            const std::vector<CombineCall>& calls, SplitMode mode,
                            cudaStream_t stream);

  // Failure record.  The kernels keep it in device memory and mirror the first failure
  // into mapped pinned host memory.  read_status() copies the device block (synchronises
  // the device, has the exact failure count); peek_status() reads the host mirror without
  // touching the device, so it also works while kernels are still waiting.
  Status read_status() const;
  Status peek_status() const;
  // Throws if the mirror holds a failure (no synchronisation: call it after the caller's own
  // stream synchronisation to cover the kernels launched so far).  With debug checks on it
  // also verifies the guard words behind every arena region (that part synchronises).
  void check_status() const;
  void verify_canaries() const;
  // After a failure the flags and counters of the protocol are in an unknown state and
  // every later dispatch() / combine() throws.  reset() clears this rank's arena, counters
  // and failure record.  It is collective by contract: every rank of the object calls it
  // once no kernel of the object is in flight anywhere, and the ranks meet at a barrier of
  // the caller's (a host barrier is enough) before the next dispatch.
  void reset();

  // Tunables (also settable through PPLX_B200_* environment variables at creation).
  void set_timeout_ms(double ms);
  void set_debug_checks(bool on) { params_.debug_checks = on ? 1 : 0; }
  // fp8 rows of this object carry power-of-two scales (see A2AParams::quant_pow2).
  void set_quant_pow2(bool on) { params_.quant_pow2 = on ? 1 : 0; }
  void set_max_blocks(int n) { max_blocks_ = n; }
  // No effect (arrival is counted in columns of the row); kept for source compatibility.
  void set_combine_units(int units);
  // Per-phase %globaltimer stamps of block 0 (see TraceSlot); synchronises on read.
  void set_trace(bool on);
  std::vector<uint64_t> read_trace() const;

  const A2AParams& params() const { return params_; }
  const SymmetricAllocation& arena() const { return *arena_; }
  const A2AConfig& config() const { return cfg_; }
  int num_local_experts() const { return params_.nle; }
  int num_dp_groups() const { return params_.num_dp_groups; }
  int experts_per_token() const { return cfg_.experts_per_token; }

  DispatchArgs make_dispatch_args(const DispatchCall& call) const;
  CombineArgs make_combine_args(const CombineCall& call) const;
  int dispatch_grid(int num_tokens) const;
  int combine_grid(int num_tokens) const;
  // Whether a dispatch of this object moves its rows as flag-in-data lines.
  bool dispatch_uses_lines(bool quantize) const;

 private:
  // The four half-operations in the only order the protocol supports.
  enum class Step { kDispatchSend = 0, kDispatchRecv = 1, kCombineSend = 2, kCombineRecv = 3 };
  void check_alive() const;
  void advance(Step step);
  // Entry of every operation: refuses a failed object, then checks and records the order.
  void begin(Step first, bool both);

  A2AConfig cfg_;
  A2AParams params_{};
  std::shared_ptr<SymmetricAllocation> arena_;
  DeviceBuffer<uint32_t> iter_;
  DeviceBuffer<uint32_t> recv_count_;
  DeviceBuffer<uint2> row_src_;
  DeviceBuffer<Status> status_;
  HostBuffer<Status> status_host_;
  std::vector<size_t> canaries_;
  Step next_ = Step::kDispatchSend;
  bool combine_send_used_lines_ = false;
  DeviceBuffer<uint64_t> trace_;
  int num_sms_ = 0;
  int max_blocks_ = 0;
};

}  // namespace pplx
