#include "all_to_all.h"

#include "../kernels/grouped_gemm.h"

#include <algorithm>
#include <sstream>

#include <nvtx3/nvToolsExt.h>

namespace pplx {

namespace {

struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
};

size_t align256(size_t x) { return round_up<size_t>(x, 256); }

const char* phase_name(uint32_t phase) {
  switch (phase) {
    case kPhaseDispatchCounts: return "dispatch: waiting for a peer's per-expert counts";
    case kPhaseDispatchPayload: return "dispatch: waiting for a peer's token payload";
    case kPhaseCombinePayload: return "combine: waiting for a token's expert outputs";
    case kPhaseBarrier: return "barrier";
    case kPhaseTest: return "wait probe";
    case kPhaseFusedGemm: return "fused expert GEMM: waiting for rows";
    default: return "unknown phase";
  }
}

const char* code_name(uint32_t code) {
  switch (code) {
    case kTimeout: return "wait timed out";
    case kBadExpert: return "expert index out of range";
    case kSlotOverflow: return "staging slot out of range";
    case kRowOverflow: return "output row out of range";
    case kBadToken: return "token index out of range";
    case kOutOfOrder: return "dispatch and combine did not alternate";
    default: return "unknown failure";
  }
}

}  // namespace

std::string describe_status(const Status& s) {
  std::ostringstream os;
  os << code_name(s.code) << " on rank " << s.rank << " (" << phase_name(s.phase)
     << "; peer/token " << s.peer << ", expected " << s.expected << ", observed " << s.observed
     << ", block " << s.block << ", " << s.count << " failure(s) in total)";
  return os.str();
}

void AllToAll::validate(const A2AConfig& c) {
  PPLX_CHECK(c.world_size >= 1 && c.world_size <= kMaxWorld,
             "world_size " << c.world_size << " not in [1, " << kMaxWorld << "]");
  PPLX_CHECK(c.rank >= 0 && c.rank < c.world_size, "rank out of range");
  PPLX_CHECK(c.dp_size >= 1 && c.world_size % c.dp_size == 0, "dp_size must divide world_size");
  PPLX_CHECK(c.max_num_tokens > 0, "max_num_tokens must be positive");
  PPLX_CHECK(c.num_experts > 0, "num_experts must be positive");
  PPLX_CHECK(c.experts_per_token > 0 && c.experts_per_token <= c.num_experts,
             "experts_per_token out of range");
  PPLX_CHECK(c.experts_per_token < (1 << 16), "experts_per_token too large");
  PPLX_CHECK(c.hidden_dim > 0, "hidden_dim must be positive");
  PPLX_CHECK(c.hidden_dim_bytes > 0 && c.hidden_dim_bytes % 16 == 0,
             "hidden_dim_bytes must be a positive multiple of 16");
  PPLX_CHECK(c.hidden_dim_scale_bytes >= 0 && c.hidden_dim_scale_bytes % 4 == 0,
             "hidden_dim_scale_bytes must be a multiple of 4");
  PPLX_CHECK(c.hidden_dim_scale_bytes <= c.hidden_dim_bytes, "scales larger than the payload");
}

namespace {

constexpr size_t kCanaryBytes = 256;
constexpr uint32_t kCanaryWord = 0xC0FFEE11u;

// Fills geometry and arena offsets; pointers stay null.  `canaries` receives the offset of
// the guard that follows each region.
A2AParams make_layout(const A2AConfig& c, std::vector<size_t>* canaries = nullptr) {
  A2AParams p{};
  p.rank = c.rank;
  p.world = c.world_size;
  p.dp_size = c.dp_size;
  p.num_dp_groups = c.world_size / c.dp_size;
  // Experts are dealt out in blocks of ceil(num_experts / world_size): expert e lives on
  // rank e / nle as local expert e % nle (the reference's rule, all_to_all.cpp:8-42).  When
  // the division leaves a remainder the last rank(s) own fewer experts; the kernels work on
  // the padded count nle * world_size, whose surplus experts simply never receive a row.
  p.nle = ceil_div(c.num_experts, c.world_size);
  p.num_experts = p.nle * c.world_size;
  p.num_real_experts = c.num_experts;
  p.topk = c.experts_per_token;
  p.max_tokens = c.max_num_tokens;
  p.hidden_dim = c.hidden_dim;
  p.hidden_bytes = c.hidden_dim_bytes;
  p.scale_bytes = c.hidden_dim_scale_bytes;
  p.trailer_off = round_up(c.hidden_dim_bytes + c.hidden_dim_scale_bytes, 16);
  // Slots start on 128-byte lines: full-line P2P writes, and TMA reads of a row
  // (fused up projection) never straddle an extra line.
  p.slot_bytes = round_up(p.trailer_off + 16, 128);
  const int tokens_per_sender = ceil_div(c.max_num_tokens, c.dp_size);
  p.region_slots = tokens_per_sender * std::min(c.experts_per_token, p.nle);
  p.cap = c.max_num_tokens * p.num_dp_groups;
  p.comb_units = c.hidden_dim;  // one arrival unit per column of an expert output row
  // Flag-in-data staging: a dispatch row is its payload lines followed by the lines of
  // its meta stream (4 trailer words, then the scales); a combine row is sized for fp32.
  p.ll_x_lines = ll::lines_for(c.hidden_dim_bytes);
  p.ll_meta_lines = ll::lines_for(16 + c.hidden_dim_scale_bytes);
  p.ll_slot_bytes = (p.ll_x_lines + p.ll_meta_lines) * ll::kLineBytes;
  p.ll_comb_slot_bytes = ll::lines_for(c.hidden_dim * 4) * ll::kLineBytes;

  // Every region is followed by a guard of kCanaryBytes that nothing may write.
  size_t off = 0;
  auto region = [&](size_t bytes) {
    const size_t at = off;
    off = align256(off + bytes);
    if (canaries != nullptr) canaries->push_back(off);
    off += kCanaryBytes;
    return at;
  };
  p.off_counts = region(sizeof(uint32_t) * 2 * p.world * p.nle);
  p.off_arrived = region(sizeof(uint32_t) * 2 * p.world);
  p.off_comb_arrived = region(sizeof(uint32_t) * p.max_tokens);
  p.off_counts_all = region(sizeof(uint32_t) * 2 * p.world * p.num_experts);
  p.off_arrived_e = region(sizeof(uint32_t) * 2 * p.nle * p.world);
  p.off_disp_stage = region(static_cast<size_t>(p.world) * p.region_slots * p.slot_bytes);
  p.off_comb_stage = region(static_cast<size_t>(p.max_tokens) * p.topk * p.hidden_dim * 4);
  p.off_ll_disp_stage = region(static_cast<size_t>(p.world) * p.region_slots * p.ll_slot_bytes);
  p.off_ll_comb_stage = region(static_cast<size_t>(p.max_tokens) * p.topk * p.ll_comb_slot_bytes);
  p.off_tiny_hdr = region(static_cast<size_t>(2) * p.world * tokens_per_sender * ll::kLineBytes);
  p.arena_bytes = off;
  return p;
}

}  // namespace

size_t AllToAll::arena_bytes(const A2AConfig& cfg) {
  validate(cfg);
  return make_layout(cfg).arena_bytes;
}

AllToAll::AllToAll(const A2AConfig& cfg, std::shared_ptr<SymmetricAllocation> arena)
    : cfg_(cfg), arena_(std::move(arena)) {
  validate(cfg_);
  params_ = make_layout(cfg_, &canaries_);
  PPLX_CHECK(arena_ && arena_->world() == cfg_.world_size && arena_->rank() == cfg_.rank,
             "arena does not match the configuration");
  PPLX_CHECK(arena_->bytes() >= params_.arena_bytes, "arena too small");
  for (int r = 0; r < cfg_.world_size; ++r) params_.peer[r] = static_cast<uint8_t*>(arena_->peer(r));
  params_.mc = static_cast<uint8_t*>(arena_->multicast());
  // Rows of replicated tokens leave once through the multicast mapping where that replaces
  // several remote copies.  On two ranks it replaces one remote and one local copy and was
  // measured slower (48 against 31 us at 128 tokens), so the default is four ranks or more;
  // PPLX_B200_MULTIMEM_COMBINE=1 / 0 forces it on / off.
  {
    const long forced = env_long("PPLX_B200_MULTIMEM_COMBINE", -1);
    const bool possible = params_.mc != nullptr && params_.dp_size == params_.world;
    params_.mc_combine = possible && (forced > 0 || (forced < 0 && params_.world >= 4)) ? 1 : 0;
  }

  iter_ = DeviceBuffer<uint32_t>(2);
  recv_count_ = DeviceBuffer<uint32_t>(params_.nle);
  row_src_ = DeviceBuffer<uint2>(static_cast<size_t>(params_.nle) * params_.cap);
  status_ = DeviceBuffer<Status>(1);
  status_host_ = HostBuffer<Status>(1, /*mapped=*/true);
  {
    Status init{};
    init.mirror = reinterpret_cast<unsigned long long>(status_host_.device_ptr());
    status_.copy_from_host(&init, 1);
  }
  trace_ = DeviceBuffer<uint64_t>(kTraceSlots);
  params_.trace = nullptr;
  params_.iter = iter_.get();
  params_.comb_iter = iter_.get() + 1;
  params_.recv_count = recv_count_.get();
  params_.row_src = row_src_.get();
  params_.status = status_.get();
  params_.timeout_ns = static_cast<uint64_t>(env_long("PPLX_B200_TIMEOUT_MS", 10000)) * 1000000ull;
  params_.debug_checks = env_long("PPLX_B200_DEBUG_CHECKS", 0) != 0 ? 1 : 0;
  // Flag-in-data lines for the plain dispatch and combine, unless switched off or the
  // object is larger than PPLX_B200_LL_MAX_TOKENS (default 512, 0 = no limit): from about a
  // thousand tokens per GPU the 6.7 % of flag bytes cost more than the fence they save.  All
  // ranks read the same environment, so they agree.
  const long ll_limit = env_long("PPLX_B200_LL_MAX_TOKENS", 512);
  params_.ll = env_long("PPLX_B200_LL", 1) != 0 &&
                       (ll_limit <= 0 || cfg_.max_num_tokens <= ll_limit)
                   ? 1
                   : 0;
  // Decode-sized objects (PPLX_B200_TINY_MAX_TOKENS, default 2, 0 = never) run the plain
  // dispatch as the header-line kernel of dispatch_tiny.cu: about 2 us faster than the general
  // kernel at one token per rank on two GPUs, level with it on eight; from four tokens on the
  // general kernel is level or ahead.
  const long tiny_limit = env_long("PPLX_B200_TINY_MAX_TOKENS", 2);
  params_.tiny = params_.ll != 0 && tiny_limit > 0 && cfg_.max_num_tokens <= tiny_limit &&
                         dispatch_tiny_supports(params_)
                     ? 1
                     : 0;
  num_sms_ = get_sm_count();
  max_blocks_ = static_cast<int>(env_long("PPLX_B200_NUM_SMS", 0));
  {
    int smem_limit = 0;
    CUDA_CHECK(cudaDeviceGetAttribute(&smem_limit, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                                      current_device()));
    PPLX_CHECK(dispatch_smem_bytes(params_) <= static_cast<size_t>(smem_limit),
               "num_experts " << cfg_.num_experts << " with world_size " << cfg_.world_size
                              << " needs " << dispatch_smem_bytes(params_)
                              << " bytes of shared memory per block for the dispatch histogram; "
                                 "the device offers "
                              << smem_limit);
  }
  // Guards after every region of this rank's arena (peers never write there).
  {
    std::vector<uint32_t> pattern(kCanaryBytes / sizeof(uint32_t), kCanaryWord);
    for (size_t at : canaries_) {
      CUDA_CHECK(cudaMemcpy(params_.peer[cfg_.rank] + at, pattern.data(), kCanaryBytes,
                            cudaMemcpyHostToDevice));
    }
  }
  CUDA_CHECK(cudaDeviceSynchronize());
}

AllToAll::~AllToAll() {
  // Kernels of this object may still be in flight on some stream.
  cudaDeviceSynchronize();
}

std::unique_ptr<AllToAll> AllToAll::create(const A2AConfig& cfg, Bootstrap& bs) {
  validate(cfg);
  PPLX_CHECK(bs.world() == cfg.world_size && bs.rank() == cfg.rank,
             "bootstrap rank/world (" << bs.rank() << "/" << bs.world()
                                      << ") differ from the configuration (" << cfg.rank << "/"
                                      << cfg.world_size << ")");
  auto arena = SymmetricAllocation::create(bs, arena_bytes(cfg));
  auto obj = std::make_unique<AllToAll>(cfg, std::move(arena));
  bs.barrier();
  return obj;
}

std::vector<std::unique_ptr<AllToAll>> AllToAll::create_local_world(const A2AConfig& cfg_in) {
  A2AConfig cfg = cfg_in;
  cfg.rank = 0;
  validate(cfg);
  auto arenas = SymmetricAllocation::create_local_world(cfg.world_size, arena_bytes(cfg));
  std::vector<std::unique_ptr<AllToAll>> out;
  for (int r = 0; r < cfg.world_size; ++r) {
    cfg.rank = r;
    out.push_back(std::make_unique<AllToAll>(cfg, arenas[r]));
  }
  return out;
}

void AllToAll::verify_canaries() const {
  std::vector<uint32_t> got(kCanaryBytes / sizeof(uint32_t));
  for (size_t n = 0; n < canaries_.size(); ++n) {
    CUDA_CHECK(cudaMemcpy(got.data(), params_.peer[cfg_.rank] + canaries_[n], kCanaryBytes,
                          cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < got.size(); ++i) {
      PPLX_CHECK(got[i] == kCanaryWord, "arena guard " << n << " of rank " << cfg_.rank
                                                       << " was overwritten at byte " << 4 * i
                                                       << " (offset " << canaries_[n]
                                                       << "): some store ran past its region");
    }
  }
}

void AllToAll::check_alive() const {
  const Status s = status_host_[0];
  if (s.code != kOk) {
    throw Error("pplx_kernels_b200: this AllToAll object recorded a failure earlier and must be "
                "destroyed or reset() on every rank before it is used again: " +
                describe_status(s));
  }
}

void AllToAll::advance(Step step) {
  auto name = [](Step s) {
    switch (s) {
      case Step::kDispatchSend: return "the send half of dispatch";
      case Step::kDispatchRecv: return "the receive half of dispatch";
      case Step::kCombineSend: return "the send half of combine";
      case Step::kCombineRecv: return "the receive half of combine";
    }
    return "?";
  };
  PPLX_CHECK(step == next_, "dispatch and combine must alternate on one object (each as one call "
                            "or as its send half followed by its receive half): this call is "
                                << name(step) << ", the object expects " << name(next_));
  next_ = static_cast<Step>((static_cast<int>(step) + 1) % 4);
}

void AllToAll::begin(Step first, bool both) {
  check_alive();
  advance(first);
  if (both) advance(static_cast<Step>(static_cast<int>(first) + 1));
}

void AllToAll::reset() {
  CUDA_CHECK(cudaDeviceSynchronize());
  uint8_t* mine = params_.peer[cfg_.rank];
  CUDA_CHECK(cudaMemset(mine, 0, params_.arena_bytes));
  {
    std::vector<uint32_t> pattern(kCanaryBytes / sizeof(uint32_t), kCanaryWord);
    for (size_t at : canaries_)
      CUDA_CHECK(cudaMemcpy(mine + at, pattern.data(), kCanaryBytes, cudaMemcpyHostToDevice));
  }
  CUDA_CHECK(cudaMemset(iter_.get(), 0, iter_.bytes()));
  CUDA_CHECK(cudaMemset(recv_count_.get(), 0, recv_count_.bytes()));
  Status init{};
  init.mirror = reinterpret_cast<unsigned long long>(status_host_.device_ptr());
  status_.copy_from_host(&init, 1);
  status_host_[0] = Status{};
  next_ = Step::kDispatchSend;
  CUDA_CHECK(cudaDeviceSynchronize());
}

void AllToAll::set_combine_units(int) {
  // Kept for callers of earlier versions: arrival is counted in columns now, so any sender
  // (a row part of the combine kernel, a column block of a GEMM epilogue) adds what it covers
  // and nothing has to be agreed beforehand.
}

void AllToAll::set_trace(bool on) { params_.trace = on ? trace_.get() : nullptr; }

std::vector<uint64_t> AllToAll::read_trace() const { return trace_.to_host(); }

void AllToAll::set_timeout_ms(double ms) {
  PPLX_CHECK(ms > 0, "timeout must be positive");
  params_.timeout_ns = static_cast<uint64_t>(ms * 1e6);
}

int AllToAll::dispatch_grid(int num_tokens) const {
  const int limit = max_blocks_ > 0 ? std::min(max_blocks_, num_sms_) : num_sms_;
  const int units = std::max(1, num_tokens) * cfg_.experts_per_token;
  return std::clamp(ceil_div(units, 4), std::min(4, limit), limit);
}

bool AllToAll::dispatch_uses_lines(bool quantize) const { return params_.ll != 0 && !quantize; }

int AllToAll::combine_grid(int num_tokens) const {
  const int limit = max_blocks_ > 0 ? std::min(max_blocks_, num_sms_) : num_sms_;
  const int warps = combine_threads() / 32;
  const int chunks = ceil_div(cfg_.hidden_dim / 8, 32);
  const int units = std::max(1, num_tokens) * std::max(cfg_.experts_per_token, chunks);
  return std::clamp(ceil_div(units, warps), std::min(4, limit), limit);
}

DispatchArgs AllToAll::make_dispatch_args(const DispatchCall& c) const {
  const A2AParams& p = params_;
  // A rank may come with no tokens at all (empty tensors have no storage).
  const bool empty = c.num_tokens == 0;
  PPLX_CHECK(c.out_num_tokens != nullptr && c.out_x.data != nullptr &&
                 (empty || (c.x.data != nullptr && c.indices != nullptr)),
             "dispatch: missing tensor");
  PPLX_CHECK(c.num_tokens >= 0 && c.num_tokens <= p.max_tokens,
             "dispatch: " << c.num_tokens << " tokens exceed max_num_tokens " << p.max_tokens);
  PPLX_CHECK(c.out_rows >= p.cap, "dispatch: out_expert_x holds "
                                      << c.out_rows << " rows per expert, need " << p.cap);
  const bool has_scale = p.scale_bytes > 0;
  if (c.quantize) {
    PPLX_CHECK(p.hidden_bytes == p.hidden_dim && p.scale_bytes == ceil_div(p.hidden_dim, 128) * 4,
               "quantising dispatch needs an object created for a 1-byte payload with one fp32 "
               "scale per 128 columns");
    PPLX_CHECK(c.out_scale.data != nullptr && c.x_scale.data == nullptr,
               "quantising dispatch takes out_expert_x_scale but no dp_x_scale");
  } else {
    PPLX_CHECK(has_scale == (c.out_scale.data != nullptr) &&
                   (empty || has_scale == (c.x_scale.data != nullptr)),
               "dispatch: scale tensors must be given exactly when hidden_dim_scale_bytes > 0");
  }
  PPLX_CHECK(reinterpret_cast<uintptr_t>(c.out_x.data) % 16 == 0 &&
                 reinterpret_cast<uintptr_t>(c.x.data) % 16 == 0 && c.out_x.stride_row % 16 == 0 &&
                 c.out_x.stride_outer % 16 == 0 && c.x.stride_row % 16 == 0,
             "dispatch: token buffers must be 16-byte aligned");
  DispatchArgs a{};
  a.p = p;
  a.out_num_tokens = c.out_num_tokens;
  a.out_x = c.out_x.data;
  a.out_x_stride_e = c.out_x.stride_outer;
  a.out_x_stride_row = c.out_x.stride_row;
  a.out_scale = c.out_scale.data;
  a.out_scale_stride_e = c.out_scale.stride_outer;
  a.out_scale_stride_row = c.out_scale.stride_row;
  a.out_scale_stride_col = c.out_scale.stride_col;
  a.x = c.x.data;
  a.x_stride_row = c.x.stride_row;
  a.x_scale = c.x_scale.data;
  a.x_scale_stride_row = c.x_scale.stride_row;
  a.x_scale_stride_col = c.x_scale.stride_col;
  a.indices = c.indices;
  a.bound_m = c.bound_m;
  a.num_tokens = c.num_tokens;
  a.quantize = c.quantize ? 1 : 0;
  a.x_on_host = c.x_on_host ? 1 : 0;
  a.stage_tokens = (c.x_on_host && params_.ll != 0 && !c.quantize) ? dispatch_stage_tokens(p) : 0;
  return a;
}

CombineArgs AllToAll::make_combine_args(const CombineCall& c) const {
  const A2AParams& p = params_;
  PPLX_CHECK(c.expert_y != nullptr &&
                 (c.num_tokens == 0 || (c.out_tokens != nullptr && c.weights != nullptr)),
             "combine: missing tensor");
  PPLX_CHECK(c.num_tokens >= 0 && c.num_tokens <= p.max_tokens,
             "combine: " << c.num_tokens << " tokens exceed max_num_tokens " << p.max_tokens);
  PPLX_CHECK(p.hidden_dim % 8 == 0, "combine: hidden_dim must be a multiple of 8");
  const int64_t in_sz = static_cast<int64_t>(dtype_size(c.in));
  PPLX_CHECK(reinterpret_cast<uintptr_t>(c.expert_y) % 16 == 0 &&
                 (c.y_stride_row * in_sz) % 16 == 0 && (c.y_stride_e * in_sz) % 16 == 0 &&
                 reinterpret_cast<uintptr_t>(c.out_tokens) % 16 == 0 &&
                 (c.out_stride_row * 2) % 16 == 0,
             "combine: buffers must be 16-byte aligned");
  CombineArgs a{};
  a.p = p;
  a.out_tokens = c.out_tokens;
  a.out_stride_row = c.out_stride_row;
  a.weights = c.weights;
  a.w_stride_row = c.w_stride_row;
  a.expert_y = c.expert_y;
  a.y_stride_e = c.y_stride_e;
  a.y_stride_row = c.y_stride_row;
  a.bound_m = c.bound_m;
  a.num_tokens = c.num_tokens;
  // Replicated tokens with a multicast mapping: the counter form, whose send multicasts rows.
  a.ll = params_.ll != 0 && params_.mc_combine == 0 ? 1 : 0;
  return a;
}

namespace {

void check_local_ranks(size_t n) {
  PPLX_CHECK(n >= 1 && n <= static_cast<size_t>(kMaxLocalRanks),
             "a group launch drives between 1 and " << kMaxLocalRanks
                                                    << " ranks of one device, got " << n);
}

}  // namespace

void AllToAll::dispatch_send_packed(const DispatchCall& call, cudaStream_t stream) {
  NvtxRange range("dispatch_send_packed");
  const DispatchArgs a = make_packed_send_args(call);
  begin(Step::kDispatchSend, false);
  CUDA_CHECK(launch_dispatch(a, true, false, dispatch_grid(call.num_tokens), stream));
}

DispatchArgs AllToAll::make_packed_send_args(const DispatchCall& c) const {
  const A2AParams& p = params_;
  PPLX_CHECK(c.num_tokens == 0 || (c.x.data != nullptr && c.indices != nullptr),
             "packed dispatch: missing tensor");
  if (c.quantize) {
    PPLX_CHECK(p.hidden_bytes == p.hidden_dim && p.scale_bytes == ceil_div(p.hidden_dim, 128) * 4,
               "the quantising packed dispatch needs an object created for a 1-byte payload "
               "with one fp32 scale per 128 columns");
  } else {
    PPLX_CHECK(p.scale_bytes == 0, "the packed dispatch carries scales only when it quantises");
  }
  PPLX_CHECK(c.num_tokens >= 0 && c.num_tokens <= p.max_tokens,
             "dispatch: " << c.num_tokens << " tokens exceed max_num_tokens " << p.max_tokens);
  PPLX_CHECK(reinterpret_cast<uintptr_t>(c.x.data) % 16 == 0 && c.x.stride_row % 16 == 0,
             "dispatch: token buffers must be 16-byte aligned");
  PPLX_CHECK(static_cast<size_t>(p.world) * p.num_experts <= 16384,
             "packed dispatch supports world_size * num_experts up to 16384");
  DispatchArgs a{};
  a.p = p;
  a.x = c.x.data;
  a.x_stride_row = c.x.stride_row;
  a.indices = c.indices;
  a.bound_m = c.bound_m;
  a.num_tokens = c.num_tokens;
  a.packed = 1;
  a.quantize = c.quantize ? 1 : 0;
  return a;
}

void AllToAll::dispatch_send_packed_group(const std::vector<AllToAll*>& ranks,
                                          const std::vector<DispatchCall>& calls,
                                          cudaStream_t stream) {
  PPLX_CHECK(!ranks.empty() && ranks.size() == calls.size(), "dispatch group: size mismatch");
  check_local_ranks(ranks.size());
  std::vector<DispatchArgs> args;
  int max_tokens = 0;
  for (size_t r = 0; r < ranks.size(); ++r) {
    args.push_back(ranks[r]->make_packed_send_args(calls[r]));
    max_tokens = std::max(max_tokens, calls[r].num_tokens);
  }
  const int n = static_cast<int>(ranks.size());
  const int grid = std::min(ranks[0]->dispatch_grid(max_tokens), std::max(1, ranks[0]->num_sms_ / n));
  for (AllToAll* r : ranks) r->begin(Step::kDispatchSend, false);
  DispatchMulti multi{};
  for (int r = 0; r < n; ++r) multi.r[r] = args[r];
  CUDA_CHECK(launch_dispatch_multi(multi, n, true, false, grid, stream));
}

void AllToAll::dispatch(const DispatchCall& call, SplitMode mode, cudaStream_t stream) {
  NvtxRange range("dispatch");
  const DispatchArgs a = make_dispatch_args(call);
  const bool send = mode != SplitMode::kRecv, recv = mode != SplitMode::kSend;
  begin(send ? Step::kDispatchSend : Step::kDispatchRecv, send && recv);
  if (params_.tiny != 0 && !call.quantize) {
    const int limit = max_blocks_ > 0 ? std::min(max_blocks_, num_sms_) : num_sms_;
    CUDA_CHECK(launch_dispatch_tiny(a, send, recv, dispatch_tiny_grid(params_, limit), stream));
    return;
  }
  CUDA_CHECK(launch_dispatch(a, send, recv, dispatch_grid(call.num_tokens), stream));
}

void AllToAll::combine(const CombineCall& call, SplitMode mode, cudaStream_t stream) {
  NvtxRange range("combine");
  CombineArgs a = make_combine_args(call);
  const bool send = mode != SplitMode::kRecv, recv = mode != SplitMode::kSend;
  begin(send ? Step::kCombineSend : Step::kCombineRecv, send && recv);
  // The receive half follows whatever its send half used: lines for a send of this class,
  // counters after the GEMM-epilogue send of the fused MoE path.
  if (send) combine_send_used_lines_ = a.ll != 0;
  else a.ll = combine_send_used_lines_ ? 1 : 0;
  CUDA_CHECK(launch_combine(a, call.in, call.out, send, recv, combine_grid(call.num_tokens),
                            stream));
}

void AllToAll::fused_up(const FusedFfnCall& f, cudaStream_t stream) {
  NvtxRange range("moe_fused_up");
  begin(Step::kDispatchRecv, false);
  GroupedGemmCall c;
  c.w = f.w;
  c.w_stride_e = f.w_stride_e;
  c.w_stride_row = f.w_stride_row;
  c.out = f.h;
  c.out_stride_e = f.h_stride_e;
  c.out_stride_row = f.h_stride_row;
  c.status = f.status;
  c.num_experts = params_.nle;
  c.rows_per_expert = f.rows_per_expert;
  c.n_out = f.inter_dim;
  c.k = params_.hidden_dim;
  c.swiglu = true;
  c.expected_total_rows = f.expected_total_rows;
  c.num_sms = max_blocks_ > 0 ? std::min(max_blocks_, num_sms_) : num_sms_;
  launch_gemm_from_staging(c, params_, f.out_num_tokens, stream);
}

void AllToAll::fused_up_fp8(const FusedFfnFp8Call& f, cudaStream_t stream) {
  NvtxRange range("moe_fused_up_fp8");
  begin(Step::kDispatchRecv, false);
  Fp8GemmCall c;
  c.w = f.w;
  c.w_stride_e = f.w_stride_e;
  c.w_stride_row = f.w_stride_row;
  c.sw = f.sw;
  c.sw_stride_e = f.sw_stride_e;
  c.sw_stride_row = f.sw_stride_row;
  c.out = f.h;
  c.out_stride_e = f.h_stride_e;
  c.out_stride_row = f.h_stride_row;
  c.out_scale = f.h_scale;
  c.os_stride_e = f.hs_stride_e;
  c.os_stride_row = f.hs_stride_row;
  c.status = f.status;
  c.num_experts = params_.nle;
  c.rows_per_expert = f.rows_per_expert;
  c.n_out = f.inter_dim;
  c.k = params_.hidden_dim;
  c.swiglu_quant = true;
  c.pow2_scales = params_.quant_pow2 != 0;
  c.num_sms = max_blocks_ > 0 ? std::min(max_blocks_, num_sms_) : num_sms_;
  launch_gemm_fp8_from_staging(c, params_, f.out_num_tokens, stream);
}

void AllToAll::fused_down_fp8(const FusedFfnFp8Call& f, cudaStream_t stream) {
  NvtxRange range("moe_fused_down_fp8");
  begin(Step::kCombineSend, false);
  combine_send_used_lines_ = false;
  Fp8GemmCall c;
  c.x = f.h;
  c.x_stride_e = f.h_stride_e;
  c.x_stride_row = f.h_stride_row;
  c.sa = f.h_scale;
  c.sa_stride_e = f.hs_stride_e;
  c.sa_stride_row = f.hs_stride_row;
  c.w = f.w;
  c.w_stride_e = f.w_stride_e;
  c.w_stride_row = f.w_stride_row;
  c.sw = f.sw;
  c.sw_stride_e = f.sw_stride_e;
  c.sw_stride_row = f.sw_stride_row;
  c.counts = reinterpret_cast<const int32_t*>(params_.recv_count);
  c.status = f.status;
  c.pow2_scales = params_.quant_pow2 != 0;
  c.num_experts = params_.nle;
  c.rows_per_expert = f.rows_per_expert;
  c.n_out = params_.hidden_dim;
  c.k = f.inter_dim;
  c.swiglu_quant = false;
  c.num_sms = max_blocks_ > 0 ? std::min(max_blocks_, num_sms_) : num_sms_;
  launch_gemm_fp8_to_peers(c, params_, stream);
}

void AllToAll::fused_down(const FusedFfnCall& f, cudaStream_t stream) {
  NvtxRange range("moe_fused_down");
  begin(Step::kCombineSend, false);
  combine_send_used_lines_ = false;
  GroupedGemmCall c;
  c.x = f.h;
  c.x_stride_e = f.h_stride_e;
  c.x_stride_row = f.h_stride_row;
  c.w = f.w;
  c.w_stride_e = f.w_stride_e;
  c.w_stride_row = f.w_stride_row;
  c.counts = reinterpret_cast<const int32_t*>(params_.recv_count);
  c.status = f.status;
  c.num_experts = params_.nle;
  c.rows_per_expert = f.rows_per_expert;
  c.n_out = params_.hidden_dim;
  c.k = f.inter_dim;
  c.swiglu = false;
  c.expected_total_rows = f.expected_total_rows;
  c.num_sms = max_blocks_ > 0 ? std::min(max_blocks_, num_sms_) : num_sms_;
  launch_gemm_to_peers(c, params_, stream);
}


void AllToAll::dispatch_group(const std::vector<AllToAll*>& ranks,
                              const std::vector<DispatchCall>& calls, SplitMode mode,
                              cudaStream_t stream) {
  PPLX_CHECK(!ranks.empty() && ranks.size() == calls.size(), "dispatch_group: size mismatch");
  check_local_ranks(ranks.size());
  std::vector<DispatchArgs> args;
  int grid = 1, max_tokens = 0;
  for (size_t r = 0; r < ranks.size(); ++r) {
    args.push_back(ranks[r]->make_dispatch_args(calls[r]));
    max_tokens = std::max(max_tokens, calls[r].num_tokens);
  }
  const int n = static_cast<int>(ranks.size());
  const int per_rank_limit = std::max(1, ranks[0]->num_sms_ / n);
  grid = std::min(ranks[0]->dispatch_grid(max_tokens), per_rank_limit);
  const bool send = mode != SplitMode::kRecv, recv = mode != SplitMode::kSend;
  for (AllToAll* r : ranks) r->begin(send ? Step::kDispatchSend : Step::kDispatchRecv, send && recv);
  DispatchMulti multi{};
  for (int r = 0; r < n; ++r) multi.r[r] = args[r];
  if (ranks[0]->params_.tiny != 0 && !calls[0].quantize) {
    const int limit = ranks[0]->max_blocks_ > 0 ? std::min(ranks[0]->max_blocks_, per_rank_limit)
                                                 : per_rank_limit;
    CUDA_CHECK(launch_dispatch_tiny_multi(multi, n, send, recv,
                                          dispatch_tiny_grid(ranks[0]->params_, limit), stream));
    return;
  }
  CUDA_CHECK(launch_dispatch_multi(multi, n, send, recv, grid, stream));
}

void AllToAll::combine_group(const std::vector<AllToAll*>& ranks,
                             const std::vector<CombineCall>& calls, SplitMode mode,
                             cudaStream_t stream) {
  PPLX_CHECK(!ranks.empty() && ranks.size() == calls.size(), "combine_group: size mismatch");
  check_local_ranks(ranks.size());
  std::vector<CombineArgs> args;
  int max_tokens = 0;
  for (size_t r = 0; r < ranks.size(); ++r) {
    args.push_back(ranks[r]->make_combine_args(calls[r]));
    max_tokens = std::max(max_tokens, calls[r].num_tokens);
    PPLX_CHECK(calls[r].in == calls[0].in && calls[r].out == calls[0].out,
               "combine_group: all ranks must use the same dtypes");
  }
  const int n = static_cast<int>(ranks.size());
  const int per_rank_limit = std::max(1, ranks[0]->num_sms_ / n);
  const int grid = std::min(ranks[0]->combine_grid(max_tokens), per_rank_limit);
  const bool send = mode != SplitMode::kRecv, recv = mode != SplitMode::kSend;
  for (size_t r = 0; r < ranks.size(); ++r) {
    ranks[r]->begin(send ? Step::kCombineSend : Step::kCombineRecv, send && recv);
    if (send) ranks[r]->combine_send_used_lines_ = args[r].ll != 0;
    else args[r].ll = ranks[r]->combine_send_used_lines_ ? 1 : 0;
  }
  CombineMulti multi{};
  for (int r = 0; r < n; ++r) multi.r[r] = args[r];
  CUDA_CHECK(launch_combine_multi(multi, n, calls[0].in, calls[0].out, send, recv, grid, stream));
}

Status AllToAll::read_status() const {
  Status s{};
  CUDA_CHECK(cudaMemcpy(&s, status_.get(), sizeof(Status), cudaMemcpyDeviceToHost));
  s.mirror = 0;
  return s;
}

Status AllToAll::peek_status() const {
  Status s = status_host_[0];
  s.mirror = 0;
  return s;
}

void AllToAll::check_status() const {
  const Status s = peek_status();
  if (s.code != kOk) throw Error("pplx_kernels_b200: " + describe_status(s));
  if (params_.debug_checks) verify_canaries();
}

}  // namespace pplx
