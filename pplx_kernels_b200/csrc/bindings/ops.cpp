// Torch operator library `pplx_kernels_b200`.
//
// Role parity: csrc/bindings/{bindings,all_to_all_ops,nvshmem}.cpp of the
// reference.  The six all-to-all operators and the ten symmetric-memory
// operators keep the reference's names, argument order and mutation
// annotations (all_to_all_ops.cpp:329-391, nvshmem.cpp:86-98), so the Python
// wrappers and torch.compile see the same surface; Meta implementations are
// no-ops.  Extra operators expose what the reference lacks: status checks,
// tunables, single-device multi-rank worlds, a sleep kernel and a wait probe.
#include <mutex>
#include <unordered_map>

#include <sys/mman.h>
#include <unistd.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/csrc/distributed/c10d/GroupRegistry.hpp>
#include <torch/csrc/distributed/c10d/ProcessGroup.hpp>
#include <torch/library.h>

#include "../core/utils.h"
#include "../kernels/collectives.h"
#include "../runtime/all_to_all.h"
#include "../runtime/bootstrap.h"
#include "../runtime/runtime.h"
#include "../runtime/vmm.h"
#include "registration.h"

namespace pplx {
namespace {

// ------------------------------------------------------------- bootstrap ----

// Blob exchange over a c10d ProcessGroup (role of DistributedTorch,
// all_to_all_ops.cpp:26-52).  CPU tensors are used when the group has a CPU
// backend (gloo); otherwise the blobs take a detour through device memory.
class TorchBootstrap final : public Bootstrap {
 public:
  explicit TorchBootstrap(c10::intrusive_ptr<c10d::ProcessGroup> group)
      : group_(std::move(group)) {}
  int rank() const override { return group_->getRank(); }
  int world() const override { return group_->getSize(); }

  void all_gather(const void* in, void* out, size_t bytes) override {
    const int64_t n = static_cast<int64_t>(bytes);
    const int64_t w = world();
    auto run = [&](const at::TensorOptions& opts) {
      at::Tensor src = at::empty({n}, at::TensorOptions().dtype(at::kByte));
      std::memcpy(src.data_ptr(), in, bytes);
      at::Tensor input = src.to(opts.device());
      at::Tensor output = at::empty({w * n}, opts);
      group_->_allgather_base(output, input)->wait();
      at::Tensor host = output.cpu();
      std::memcpy(out, host.data_ptr(), bytes * w);
    };
    bool done = false;
    if (!force_cuda_) {
      try {
        run(at::TensorOptions().dtype(at::kByte).device(at::kCPU));
        done = true;
      } catch (const std::exception&) {
        force_cuda_ = true;
      }
    }
    if (!done) run(at::TensorOptions().dtype(at::kByte).device(at::kCUDA, current_device()));
  }

 private:
  c10::intrusive_ptr<c10d::ProcessGroup> group_;
  bool force_cuda_ = false;
};

// ---------------------------------------------------------- object table ----

std::mutex g_mu;
std::unordered_map<int64_t, std::unique_ptr<AllToAll>> g_objects;

int64_t adopt(std::unique_ptr<AllToAll> obj) {
  const int64_t key = reinterpret_cast<int64_t>(obj.get());
  std::lock_guard<std::mutex> lock(g_mu);
  g_objects[key] = std::move(obj);
  return key;
}

AllToAll* lookup(int64_t ptr) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_objects.find(ptr);
  TORCH_CHECK(it != g_objects.end(), "invalid or destroyed AllToAll handle");
  return it->second.get();
}

A2AConfig make_config(int64_t max_num_tokens, int64_t num_experts, int64_t experts_per_token,
                      int64_t rank, int64_t world_size, int64_t dp_size, int64_t hidden_dim,
                      int64_t hidden_dim_bytes, int64_t hidden_dim_scale_bytes) {
  A2AConfig c;
  c.max_num_tokens = static_cast<int>(max_num_tokens);
  c.num_experts = static_cast<int>(num_experts);
  c.experts_per_token = static_cast<int>(experts_per_token);
  c.rank = static_cast<int>(rank);
  c.world_size = static_cast<int>(world_size);
  c.dp_size = static_cast<int>(dp_size);
  c.hidden_dim = static_cast<int>(hidden_dim);
  c.hidden_dim_bytes = static_cast<int>(hidden_dim_bytes);
  c.hidden_dim_scale_bytes = static_cast<int>(hidden_dim_scale_bytes);
  return c;
}

template <typename F>
auto guarded(F&& fn) -> decltype(fn()) {
  try {
    return fn();
  } catch (const Error& e) {
    TORCH_CHECK(false, e.what());
  }
}

int64_t create_intranode(int64_t max_num_tokens, int64_t num_experts, int64_t experts_per_token,
                         int64_t rank, int64_t world_size, int64_t dp_size, int64_t hidden_dim,
                         int64_t hidden_dim_bytes, int64_t hidden_dim_scale_bytes,
                         const std::string& group_name) {
  return guarded([&] {
    const A2AConfig cfg =
        make_config(max_num_tokens, num_experts, experts_per_token, rank, world_size, dp_size,
                    hidden_dim, hidden_dim_bytes, hidden_dim_scale_bytes);
    AllToAll::validate(cfg);
    if (world_size == 1) {
      SingleBootstrap bs;
      return adopt(AllToAll::create(cfg, bs));
    }
    TorchBootstrap bs(c10d::resolve_process_group(group_name));
    return adopt(AllToAll::create(cfg, bs));
  });
}

int64_t create_internode(int64_t max_num_tokens, int64_t num_experts, int64_t experts_per_token,
                         int64_t rank, int64_t world_size, int64_t dp_size, int64_t hidden_dim,
                         int64_t hidden_dim_bytes, int64_t hidden_dim_scale_bytes) {
  return guarded([&] {
    const A2AConfig cfg =
        make_config(max_num_tokens, num_experts, experts_per_token, rank, world_size, dp_size,
                    hidden_dim, hidden_dim_bytes, hidden_dim_scale_bytes);
    AllToAll::validate(cfg);
    return adopt(AllToAll::create(cfg, Runtime::instance().bootstrap()));
  });
}

std::vector<int64_t> create_local_world(int64_t max_num_tokens, int64_t num_experts,
                                        int64_t experts_per_token, int64_t world_size,
                                        int64_t dp_size, int64_t hidden_dim,
                                        int64_t hidden_dim_bytes,
                                        int64_t hidden_dim_scale_bytes) {
  return guarded([&] {
    const A2AConfig cfg = make_config(max_num_tokens, num_experts, experts_per_token, 0,
                                      world_size, dp_size, hidden_dim, hidden_dim_bytes,
                                      hidden_dim_scale_bytes);
    std::vector<int64_t> out;
    for (auto& obj : AllToAll::create_local_world(cfg)) out.push_back(adopt(std::move(obj)));
    return out;
  });
}

void destroy(int64_t ptr) {
  std::unique_ptr<AllToAll> victim;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_objects.find(ptr);
    if (it == g_objects.end()) return;
    victim = std::move(it->second);
    g_objects.erase(it);
  }
  victim.reset();
}

// ------------------------------------------------------------ tensor glue ----

// Inputs may live in pinned host memory instead of device memory (an extension over the
// reference): the kernels then read them across PCIe themselves and no upload precedes
// the call.  Returns the address the device uses for `t`.
bool on_pinned_host(const at::Tensor& t) { return t.is_cpu() && t.is_pinned(); }

const void* device_address(const at::Tensor& t, const char* name) {
  if (t.is_cuda()) return t.data_ptr();
  TORCH_CHECK(on_pinned_host(t), name, " must be a CUDA tensor or a pinned host tensor");
  if (t.numel() == 0) return nullptr;
  void* mapped = nullptr;
  const cudaError_t err = cudaHostGetDevicePointer(&mapped, t.data_ptr(), 0);
  TORCH_CHECK(err == cudaSuccess, name, ": pinned memory is not mapped into the device (",
              cudaGetErrorString(err), ")");
  return mapped;
}

DispatchCall make_dispatch_call(const AllToAll& ata, at::Tensor& out_expert_num_tokens,
                                at::Tensor& out_expert_x,
                                const std::optional<at::Tensor>& out_expert_x_scale,
                                const at::Tensor& dp_x, const std::optional<at::Tensor>& dp_x_scale,
                                const at::Tensor& indices,
                                const std::optional<at::Tensor>& bound_m,
                                bool quantize = false) {
  const A2AParams& p = ata.params();
  TORCH_CHECK(out_expert_num_tokens.is_cuda() && out_expert_num_tokens.dim() == 1 &&
                  out_expert_num_tokens.scalar_type() == at::kInt &&
                  out_expert_num_tokens.is_contiguous() &&
                  out_expert_num_tokens.size(0) == p.nle,
              "out_expert_num_tokens must be a contiguous int32 CUDA tensor of [num_local_experts]");
  TORCH_CHECK(out_expert_x.is_cuda() && out_expert_x.dim() == 3 && out_expert_x.is_contiguous(),
              "out_expert_x must be a contiguous 3-D CUDA tensor");
  TORCH_CHECK(out_expert_x.size(0) == p.nle, "out_expert_x.size(0) must be num_local_experts");
  TORCH_CHECK(out_expert_x.size(2) * static_cast<int64_t>(out_expert_x.element_size()) ==
                  p.hidden_bytes,
              "out_expert_x rows must be hidden_dim_bytes long");
  const bool host_in = on_pinned_host(dp_x);
  TORCH_CHECK((dp_x.is_cuda() || host_in) && dp_x.dim() == 2 && dp_x.is_contiguous(),
              "dp_x must be a contiguous 2-D CUDA (or pinned host) tensor");
  if (quantize) {
    TORCH_CHECK(dp_x.scalar_type() == at::kBFloat16 && dp_x.size(1) == p.hidden_dim,
                "quantising dispatch takes bfloat16 tokens of [num_tokens, hidden_dim]");
  } else {
    TORCH_CHECK(dp_x.size(1) * static_cast<int64_t>(dp_x.element_size()) == p.hidden_bytes,
                "dp_x rows must be hidden_dim_bytes long");
  }
  // Every block reads the whole routing table, so with the tokens in host memory it is
  // cheaper to keep `indices` (a few KiB) on the device; both are accepted.
  TORCH_CHECK((indices.is_cuda() || (host_in && on_pinned_host(indices))) && indices.dim() == 2 &&
                  indices.is_contiguous() && indices.element_size() == 4 &&
                  indices.size(1) == p.topk,
              "indices must be a contiguous 32-bit tensor of [num_tokens, experts_per_token] on "
              "the device (or, with dp_x in pinned host memory, in pinned host memory too)");
  TORCH_CHECK(indices.size(0) == dp_x.size(0), "indices and dp_x disagree on the token count");

  DispatchCall c;
  c.x_on_host = host_in;
  c.out_num_tokens = out_expert_num_tokens.data_ptr<int32_t>();
  c.out_x.data = static_cast<uint8_t*>(out_expert_x.data_ptr());
  c.out_x.stride_outer = out_expert_x.stride(0) * out_expert_x.element_size();
  c.out_x.stride_row = out_expert_x.stride(1) * out_expert_x.element_size();
  c.out_rows = out_expert_x.size(1);
  c.x.data = static_cast<const uint8_t*>(device_address(dp_x, "dp_x"));
  c.x.stride_row = dp_x.stride(0) * dp_x.element_size();
  if (out_expert_x_scale.has_value()) {
    const at::Tensor& s = *out_expert_x_scale;
    TORCH_CHECK(s.is_cuda() && s.dim() == 3 && s.scalar_type() == at::kFloat,
                "out_expert_x_scale must be a 3-D float32 CUDA tensor");
    TORCH_CHECK(s.size(0) == p.nle && s.size(1) == out_expert_x.size(1) &&
                    s.size(2) * 4 == p.scale_bytes,
                "out_expert_x_scale has the wrong shape");
    c.out_scale.data = s.data_ptr<float>();
    c.out_scale.stride_outer = s.stride(0);
    c.out_scale.stride_row = s.stride(1);
    c.out_scale.stride_col = s.stride(2);
  }
  if (dp_x_scale.has_value()) {
    const at::Tensor& s = *dp_x_scale;
    TORCH_CHECK((host_in ? on_pinned_host(s) : s.is_cuda()) && s.dim() == 2 &&
                    s.scalar_type() == at::kFloat,
                "dp_x_scale must be a 2-D float32 tensor in the same kind of memory as dp_x");
    TORCH_CHECK(s.size(0) == dp_x.size(0) && s.size(1) * 4 == p.scale_bytes,
                "dp_x_scale has the wrong shape");
    c.x_scale.data = static_cast<const float*>(device_address(s, "dp_x_scale"));
    c.x_scale.stride_row = s.stride(0);
    c.x_scale.stride_col = s.stride(1);
  }
  c.indices = static_cast<const uint32_t*>(device_address(indices, "indices"));
  if (bound_m.has_value()) {
    TORCH_CHECK(bound_m->is_cuda() && bound_m->numel() == 1 && bound_m->element_size() == 4,
                "bound_m must be a 32-bit CUDA scalar tensor");
    c.bound_m = static_cast<const uint32_t*>(bound_m->data_ptr());
  }
  c.num_tokens = static_cast<int>(indices.size(0));
  c.quantize = quantize;
  return c;
}

DType to_dtype(at::ScalarType t, const char* what) {
  switch (t) {
    case at::kFloat: return DType::kF32;
    case at::kHalf: return DType::kF16;
    case at::kBFloat16: return DType::kBF16;
    default: TORCH_CHECK(false, what, ": unsupported dtype ", t);
  }
}

CombineCall make_combine_call(const AllToAll& ata, at::Tensor& out_tokens,
                              const at::Tensor& indices, const at::Tensor& weights,
                              const at::Tensor& expert_y,
                              const std::optional<at::Tensor>& bound_m) {
  const A2AParams& p = ata.params();
  // Extension over the reference: out_tokens may live in pinned host memory; the
  // reduction then writes its result across PCIe itself and no copy follows.
  const bool host_out = out_tokens.is_cpu() && out_tokens.is_pinned();
  TORCH_CHECK((out_tokens.is_cuda() || host_out) && out_tokens.dim() == 2 &&
                  out_tokens.stride(1) == 1 && out_tokens.size(1) == p.hidden_dim,
              "out_tokens must be a CUDA (or pinned host) tensor of [*, hidden_dim] with unit "
              "column stride");
  TORCH_CHECK(out_tokens.scalar_type() == at::kHalf || out_tokens.scalar_type() == at::kBFloat16,
              "out_tokens must be float16 or bfloat16");
  TORCH_CHECK((indices.is_cuda() || on_pinned_host(indices)) && indices.dim() == 2 &&
                  indices.size(1) == p.topk,
              "indices must be a CUDA (or pinned host) tensor of [num_tokens, experts_per_token]");
  TORCH_CHECK((weights.is_cuda() || on_pinned_host(weights)) && weights.dim() == 2 &&
                  weights.scalar_type() == at::kFloat && weights.stride(1) == 1 &&
                  weights.size(0) == indices.size(0) && weights.size(1) == p.topk,
              "weights must be a float32 CUDA (or pinned host) tensor of [num_tokens, "
              "experts_per_token]");
  TORCH_CHECK(out_tokens.size(0) >= indices.size(0), "out_tokens has fewer rows than indices");
  TORCH_CHECK(expert_y.is_cuda() && expert_y.dim() == 3 && expert_y.stride(2) == 1 &&
                  expert_y.size(0) == p.nle && expert_y.size(1) >= p.cap &&
                  expert_y.size(2) == p.hidden_dim,
              "expert_y must be a CUDA tensor of [num_local_experts, max_num_tokens * "
              "num_dp_groups, hidden_dim]");
  CombineCall c;
  c.out_tokens = out_tokens.data_ptr();
  if (host_out) {
    void* mapped = nullptr;
    const cudaError_t err = cudaHostGetDevicePointer(&mapped, out_tokens.data_ptr(), 0);
    TORCH_CHECK(err == cudaSuccess, "out_tokens: pinned memory is not mapped into the device (",
                cudaGetErrorString(err), ")");
    c.out_tokens = mapped;
  }
  c.out_stride_row = out_tokens.stride(0);
  c.weights = static_cast<const float*>(device_address(weights, "weights"));
  c.w_stride_row = weights.stride(0);
  c.expert_y = expert_y.data_ptr();
  c.y_stride_e = expert_y.stride(0);
  c.y_stride_row = expert_y.stride(1);
  if (bound_m.has_value()) {
    TORCH_CHECK(bound_m->is_cuda() && bound_m->numel() == 1 && bound_m->element_size() == 4,
                "bound_m must be a 32-bit CUDA scalar tensor");
    c.bound_m = static_cast<const uint32_t*>(bound_m->data_ptr());
  }
  c.num_tokens = static_cast<int>(indices.size(0));
  c.in = to_dtype(expert_y.scalar_type(), "expert_y");
  c.out = to_dtype(out_tokens.scalar_type(), "out_tokens");
  return c;
}

void dispatch_op(int64_t ptr, at::Tensor& out_expert_num_tokens, at::Tensor& out_expert_x,
                 const std::optional<at::Tensor>& out_expert_x_scale, const at::Tensor& dp_x,
                 const std::optional<at::Tensor>& dp_x_scale, const at::Tensor& indices,
                 const std::optional<at::Tensor>& bound_m, bool do_send, bool do_recv) {
  AllToAll* ata = lookup(ptr);
  const c10::cuda::OptionalCUDAGuard guard(out_expert_x.device());
  guarded([&] {
    const DispatchCall call = make_dispatch_call(*ata, out_expert_num_tokens, out_expert_x,
                                                 out_expert_x_scale, dp_x, dp_x_scale, indices,
                                                 bound_m);
    ata->dispatch(call, split_mode(do_send, do_recv), at::cuda::getCurrentCUDAStream());
  });
}

// dispatch with the bf16 -> fp8 (e4m3, fp32 scale per 128 columns) conversion fused
// into the send.  No counterpart in the reference, which never interprets the payload.
void dispatch_quant_op(int64_t ptr, at::Tensor& out_expert_num_tokens, at::Tensor& out_expert_x,
                       at::Tensor& out_expert_x_scale, const at::Tensor& dp_x,
                       const at::Tensor& indices, const std::optional<at::Tensor>& bound_m,
                       bool do_send, bool do_recv) {
  AllToAll* ata = lookup(ptr);
  const c10::cuda::OptionalCUDAGuard guard(out_expert_x.device());
  guarded([&] {
    const DispatchCall call =
        make_dispatch_call(*ata, out_expert_num_tokens, out_expert_x, out_expert_x_scale, dp_x,
                           std::nullopt, indices, bound_m, /*quantize=*/true);
    ata->dispatch(call, split_mode(do_send, do_recv), at::cuda::getCurrentCUDAStream());
  });
}

void fake_dispatch_quant(int64_t, at::Tensor&, at::Tensor&, at::Tensor&, const at::Tensor&,
                         const at::Tensor&, const std::optional<at::Tensor>&, bool, bool) {}

void combine_op(int64_t ptr, at::Tensor& out_tokens, const at::Tensor& indices,
                const at::Tensor& weights, const at::Tensor& expert_y,
                const std::optional<at::Tensor>& bound_m, bool do_send, bool do_recv) {
  AllToAll* ata = lookup(ptr);
  const c10::cuda::OptionalCUDAGuard guard(expert_y.device());
  guarded([&] {
    const CombineCall call = make_combine_call(*ata, out_tokens, indices, weights, expert_y, bound_m);
    ata->combine(call, split_mode(do_send, do_recv), at::cuda::getCurrentCUDAStream());
  });
}

void fake_dispatch(int64_t, at::Tensor&, at::Tensor&, const std::optional<at::Tensor>&,
                   const at::Tensor&, const std::optional<at::Tensor>&, const at::Tensor&,
                   const std::optional<at::Tensor>&, bool, bool) {}

void fake_combine(int64_t, at::Tensor&, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                  const std::optional<at::Tensor>&, bool, bool) {}

std::optional<at::Tensor> opt(const at::Tensor& t) {
  return t.numel() == 0 ? std::nullopt : std::optional<at::Tensor>(t);
}

// Group launches take parallel lists; an empty tensor stands for "None".
void dispatch_group_op(std::vector<int64_t> ptrs, std::vector<at::Tensor> out_expert_num_tokens,
                       std::vector<at::Tensor> out_expert_x,
                       std::vector<at::Tensor> out_expert_x_scale, std::vector<at::Tensor> dp_x,
                       std::vector<at::Tensor> dp_x_scale, std::vector<at::Tensor> indices,
                       std::vector<at::Tensor> bound_m, bool do_send, bool do_recv) {
  const size_t n = ptrs.size();
  TORCH_CHECK(n > 0 && out_expert_num_tokens.size() == n && out_expert_x.size() == n &&
                  out_expert_x_scale.size() == n && dp_x.size() == n && dp_x_scale.size() == n &&
                  indices.size() == n && bound_m.size() == n,
              "dispatch_group: list lengths differ");
  guarded([&] {
    std::vector<AllToAll*> ranks;
    std::vector<DispatchCall> calls;
    for (size_t r = 0; r < n; ++r) {
      ranks.push_back(lookup(ptrs[r]));
      calls.push_back(make_dispatch_call(*ranks[r], out_expert_num_tokens[r], out_expert_x[r],
                                         opt(out_expert_x_scale[r]), dp_x[r], opt(dp_x_scale[r]),
                                         indices[r], opt(bound_m[r])));
    }
    const c10::cuda::OptionalCUDAGuard guard(dp_x[0].device());
    AllToAll::dispatch_group(ranks, calls, split_mode(do_send, do_recv),
                             at::cuda::getCurrentCUDAStream());
  });
}

void dispatch_quant_group_op(std::vector<int64_t> ptrs,
                             std::vector<at::Tensor> out_expert_num_tokens,
                             std::vector<at::Tensor> out_expert_x,
                             std::vector<at::Tensor> out_expert_x_scale,
                             std::vector<at::Tensor> dp_x, std::vector<at::Tensor> indices,
                             std::vector<at::Tensor> bound_m) {
  const size_t n = ptrs.size();
  TORCH_CHECK(n > 0 && out_expert_num_tokens.size() == n && out_expert_x.size() == n &&
                  out_expert_x_scale.size() == n && dp_x.size() == n && indices.size() == n &&
                  bound_m.size() == n,
              "dispatch_quant_group: list lengths differ");
  guarded([&] {
    std::vector<AllToAll*> ranks;
    std::vector<DispatchCall> calls;
    for (size_t r = 0; r < n; ++r) {
      ranks.push_back(lookup(ptrs[r]));
      calls.push_back(make_dispatch_call(*ranks[r], out_expert_num_tokens[r], out_expert_x[r],
                                         out_expert_x_scale[r], dp_x[r], std::nullopt, indices[r],
                                         opt(bound_m[r]), /*quantize=*/true));
    }
    const c10::cuda::OptionalCUDAGuard guard(dp_x[0].device());
    AllToAll::dispatch_group(ranks, calls, SplitMode::kNone, at::cuda::getCurrentCUDAStream());
  });
}

void combine_group_op(std::vector<int64_t> ptrs, std::vector<at::Tensor> out_tokens,
                      std::vector<at::Tensor> indices, std::vector<at::Tensor> weights,
                      std::vector<at::Tensor> expert_y, std::vector<at::Tensor> bound_m,
                      bool do_send, bool do_recv) {
  const size_t n = ptrs.size();
  TORCH_CHECK(n > 0 && out_tokens.size() == n && indices.size() == n && weights.size() == n &&
                  expert_y.size() == n && bound_m.size() == n,
              "combine_group: list lengths differ");
  guarded([&] {
    std::vector<AllToAll*> ranks;
    std::vector<CombineCall> calls;
    for (size_t r = 0; r < n; ++r) {
      ranks.push_back(lookup(ptrs[r]));
      calls.push_back(make_combine_call(*ranks[r], out_tokens[r], indices[r], weights[r],
                                        expert_y[r], opt(bound_m[r])));
    }
    const c10::cuda::OptionalCUDAGuard guard(expert_y[0].device());
    AllToAll::combine_group(ranks, calls, split_mode(do_send, do_recv),
                            at::cuda::getCurrentCUDAStream());
  });
}

// ----------------------------------------------------- status / tunables ----

std::vector<int64_t> status_op(int64_t ptr) {
  const Status s = guarded([&] { return lookup(ptr)->read_status(); });
  return {s.code, s.phase, s.peer, s.expected, s.observed, s.block, s.rank, s.count};
}

// The host-visible mirror of the failure record: no device synchronisation.
std::vector<int64_t> peek_status_op(int64_t ptr) {
  const Status s = lookup(ptr)->peek_status();
  return {s.code, s.phase, s.peer, s.expected, s.observed, s.block, s.rank, s.count};
}

void reset_op(int64_t ptr) {
  guarded([&] { lookup(ptr)->reset(); });
}

void verify_canaries_op(int64_t ptr) {
  guarded([&] { lookup(ptr)->verify_canaries(); });
}

void check_status_op(int64_t ptr) {
  guarded([&] { lookup(ptr)->check_status(); });
}

void set_timeout_ms_op(int64_t ptr, double ms) {
  guarded([&] { lookup(ptr)->set_timeout_ms(ms); });
}

void set_debug_checks_op(int64_t ptr, bool on) { lookup(ptr)->set_debug_checks(on); }
void set_quant_pow2_op(int64_t ptr, bool on) { lookup(ptr)->set_quant_pow2(on); }

void set_max_blocks_op(int64_t ptr, int64_t n) { lookup(ptr)->set_max_blocks(static_cast<int>(n)); }

void set_combine_units_op(int64_t ptr, int64_t units) {
  guarded([&] { lookup(ptr)->set_combine_units(static_cast<int>(units)); });
}

uint32_t* status_word(const std::optional<at::Tensor>& status) {
  if (!status.has_value()) return nullptr;
  TORCH_CHECK(status->is_cuda() && status->element_size() == 4 && status->numel() >= 1,
              "status must be a 32-bit CUDA tensor");
  return static_cast<uint32_t*>(status->data_ptr());
}

void check_bf16_3d(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 3 && t.scalar_type() == at::kBFloat16 && t.stride(2) == 1,
              name, " must be a 3-D bfloat16 CUDA tensor with a contiguous last dimension");
}

DispatchCall make_packed_call(const AllToAll& ata, const at::Tensor& dp_x,
                              const at::Tensor& indices,
                              const std::optional<at::Tensor>& bound_m, bool quantize = false) {
  const A2AParams& p = ata.params();
  TORCH_CHECK(dp_x.is_cuda() && dp_x.dim() == 2 && dp_x.is_contiguous() &&
                  dp_x.scalar_type() == at::kBFloat16 && dp_x.size(1) == p.hidden_dim,
              "dp_x must be a contiguous bfloat16 CUDA tensor of [num_tokens, hidden_dim]");
  TORCH_CHECK(indices.is_cuda() && indices.dim() == 2 && indices.is_contiguous() &&
                  indices.element_size() == 4 && indices.size(1) == p.topk &&
                  indices.size(0) == dp_x.size(0),
              "indices must be a contiguous 32-bit CUDA tensor of [num_tokens, experts_per_token]");
  DispatchCall c;
  c.x.data = static_cast<const uint8_t*>(dp_x.data_ptr());
  c.x.stride_row = dp_x.stride(0) * dp_x.element_size();
  c.indices = static_cast<const uint32_t*>(indices.data_ptr());
  if (bound_m.has_value()) {
    TORCH_CHECK(bound_m->is_cuda() && bound_m->numel() == 1 && bound_m->element_size() == 4,
                "bound_m must be a 32-bit CUDA scalar tensor");
    c.bound_m = static_cast<const uint32_t*>(bound_m->data_ptr());
  }
  c.num_tokens = static_cast<int>(indices.size(0));
  c.quantize = quantize;
  return c;
}

// Send half of the fused MoE dispatch: rows land in the peers' staging grouped by expert.
// With `quantize` the bf16 tokens travel as e4m3 + one fp32 scale per 128 columns.
void moe_dispatch_send_op(int64_t ptr, const at::Tensor& dp_x, const at::Tensor& indices,
                          const std::optional<at::Tensor>& bound_m, bool quantize) {
  AllToAll* ata = lookup(ptr);
  const c10::cuda::OptionalCUDAGuard guard(dp_x.device());
  guarded([&] {
    ata->dispatch_send_packed(make_packed_call(*ata, dp_x, indices, bound_m, quantize),
                              at::cuda::getCurrentCUDAStream());
  });
}

void fake_moe_dispatch_send(int64_t, const at::Tensor&, const at::Tensor&,
                            const std::optional<at::Tensor>&, bool) {}

void moe_dispatch_send_group_op(std::vector<int64_t> ptrs, std::vector<at::Tensor> dp_x,
                                std::vector<at::Tensor> indices, std::vector<at::Tensor> bound_m,
                                bool quantize) {
  const size_t n = ptrs.size();
  TORCH_CHECK(n > 0 && dp_x.size() == n && indices.size() == n && bound_m.size() == n,
              "moe_dispatch_send_group: list lengths differ");
  guarded([&] {
    std::vector<AllToAll*> ranks;
    std::vector<DispatchCall> calls;
    for (size_t r = 0; r < n; ++r) {
      ranks.push_back(lookup(ptrs[r]));
      calls.push_back(make_packed_call(*ranks[r], dp_x[r], indices[r], opt(bound_m[r]), quantize));
    }
    const c10::cuda::OptionalCUDAGuard guard(dp_x[0].device());
    AllToAll::dispatch_send_packed_group(ranks, calls, at::cuda::getCurrentCUDAStream());
  });
}

// SwiGLU up projection fed from the dispatch staging arena (after dispatch with do_recv=False).
void moe_fused_up_op(int64_t ptr, const at::Tensor& w13, at::Tensor& h,
                     const std::optional<at::Tensor>& out_expert_num_tokens,
                     const std::optional<at::Tensor>& status, int64_t expected_rows) {
  AllToAll* ata = lookup(ptr);
  check_bf16_3d(w13, "w13");
  check_bf16_3d(h, "h");
  const A2AParams& p = ata->params();
  TORCH_CHECK(w13.size(0) == p.nle && w13.size(2) == p.hidden_dim && w13.size(1) == 2 * h.size(2),
              "w13 must be [num_local_experts, 2 * intermediate, hidden]");
  TORCH_CHECK(h.size(0) == p.nle && h.size(1) >= p.cap, "h must be [num_local_experts, rows, intermediate]");
  FusedFfnCall f;
  f.w = w13.data_ptr();
  f.w_stride_e = w13.stride(0);
  f.w_stride_row = w13.stride(1);
  f.h = h.data_ptr();
  f.h_stride_e = h.stride(0);
  f.h_stride_row = h.stride(1);
  f.rows_per_expert = static_cast<int>(h.size(1));
  f.inter_dim = static_cast<int>(h.size(2));
  if (out_expert_num_tokens.has_value()) {
    TORCH_CHECK(out_expert_num_tokens->is_cuda() && out_expert_num_tokens->scalar_type() == at::kInt &&
                    out_expert_num_tokens->numel() == p.nle && out_expert_num_tokens->is_contiguous(),
                "out_expert_num_tokens must be a contiguous int32 CUDA tensor of [num_local_experts]");
    f.out_num_tokens = out_expert_num_tokens->data_ptr<int32_t>();
  }
  f.status = status_word(status);
  f.expected_total_rows = expected_rows;
  const c10::cuda::OptionalCUDAGuard guard(h.device());
  guarded([&] { ata->fused_up(f, at::cuda::getCurrentCUDAStream()); });
}

// Down projection whose epilogue stores to the tokens' home ranks (before combine with do_send=False).
void moe_fused_down_op(int64_t ptr, const at::Tensor& h, const at::Tensor& w2,
                       const std::optional<at::Tensor>& status, int64_t expected_rows) {
  AllToAll* ata = lookup(ptr);
  check_bf16_3d(w2, "w2");
  check_bf16_3d(h, "h");
  const A2AParams& p = ata->params();
  TORCH_CHECK(w2.size(0) == p.nle && w2.size(1) == p.hidden_dim && w2.size(2) == h.size(2),
              "w2 must be [num_local_experts, hidden, intermediate]");
  TORCH_CHECK(h.size(0) == p.nle && h.size(1) >= p.cap, "h must be [num_local_experts, rows, intermediate]");
  FusedFfnCall f;
  f.w = w2.data_ptr();
  f.w_stride_e = w2.stride(0);
  f.w_stride_row = w2.stride(1);
  f.h = h.data_ptr();
  f.h_stride_e = h.stride(0);
  f.h_stride_row = h.stride(1);
  f.rows_per_expert = static_cast<int>(h.size(1));
  f.inter_dim = static_cast<int>(h.size(2));
  f.status = status_word(status);
  f.expected_total_rows = expected_rows;
  const c10::cuda::OptionalCUDAGuard guard(h.device());
  guarded([&] { ata->fused_down(f, at::cuda::getCurrentCUDAStream()); });
}

void check_fp8_3d(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 3 && t.element_size() == 1 && t.stride(2) == 1, name,
              " must be a 3-D one-byte (e4m3) CUDA tensor with a contiguous last dimension");
}

void check_scale_3d(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 3 && t.scalar_type() == at::kFloat && t.stride(2) == 1,
              name, " must be a 3-D float32 CUDA tensor with a contiguous last dimension");
}

FusedFfnFp8Call make_fp8_ffn_call(const AllToAll& ata, const at::Tensor& w, const at::Tensor& sw,
                                  const at::Tensor& h, const at::Tensor& h_scale, bool up,
                                  const std::optional<at::Tensor>& status) {
  const A2AParams& p = ata.params();
  check_fp8_3d(w, "w");
  check_fp8_3d(h, "h");
  check_scale_3d(sw, "w_scale");
  check_scale_3d(h_scale, "h_scale");
  const int64_t inter = h.size(2);
  const int64_t w_rows = up ? 2 * inter : p.hidden_dim;
  const int64_t k = up ? p.hidden_dim : inter;
  TORCH_CHECK(w.size(0) == p.nle && w.size(1) == w_rows && w.size(2) == k,
              "w must be [num_local_experts, ", up ? "2 * intermediate, hidden]" : "hidden, intermediate]");
  TORCH_CHECK(sw.size(0) == p.nle && sw.size(1) == (w_rows + 127) / 128 && sw.size(2) == (k + 127) / 128,
              "w_scale must hold one value per 128 x 128 block of w");
  TORCH_CHECK(h.size(0) == p.nle && h.size(1) >= p.cap && inter % 128 == 0,
              "h must be [num_local_experts, rows, intermediate] with intermediate % 128 == 0");
  TORCH_CHECK(h_scale.size(0) == p.nle && h_scale.size(1) == h.size(1) && h_scale.size(2) == inter / 128,
              "h_scale must be [num_local_experts, rows, intermediate / 128]");
  FusedFfnFp8Call f;
  f.w = w.data_ptr();
  f.w_stride_e = w.stride(0);
  f.w_stride_row = w.stride(1);
  f.sw = sw.data_ptr<float>();
  f.sw_stride_e = sw.stride(0);
  f.sw_stride_row = sw.stride(1);
  f.h = h.data_ptr();
  f.h_stride_e = h.stride(0);
  f.h_stride_row = h.stride(1);
  f.h_scale = h_scale.data_ptr<float>();
  f.hs_stride_e = h_scale.stride(0);
  f.hs_stride_row = h_scale.stride(1);
  f.rows_per_expert = static_cast<int>(h.size(1));
  f.inter_dim = static_cast<int>(inter);
  f.status = status_word(status);
  return f;
}

// fp8 SwiGLU up projection fed from the staging arena (after moe_dispatch_send with quantize).
void moe_fused_up_fp8_op(int64_t ptr, const at::Tensor& w13, const at::Tensor& w13_scale,
                         at::Tensor& h, at::Tensor& h_scale,
                         const std::optional<at::Tensor>& out_expert_num_tokens,
                         const std::optional<at::Tensor>& status) {
  AllToAll* ata = lookup(ptr);
  FusedFfnFp8Call f = make_fp8_ffn_call(*ata, w13, w13_scale, h, h_scale, true, status);
  if (out_expert_num_tokens.has_value()) {
    TORCH_CHECK(out_expert_num_tokens->is_cuda() && out_expert_num_tokens->scalar_type() == at::kInt &&
                    out_expert_num_tokens->numel() == ata->params().nle &&
                    out_expert_num_tokens->is_contiguous(),
                "out_expert_num_tokens must be a contiguous int32 CUDA tensor of [num_local_experts]");
    f.out_num_tokens = out_expert_num_tokens->data_ptr<int32_t>();
  }
  const c10::cuda::OptionalCUDAGuard guard(h.device());
  guarded([&] { ata->fused_up_fp8(f, at::cuda::getCurrentCUDAStream()); });
}

// fp8 down projection whose epilogue stores the bf16 rows to the tokens' home ranks.
void moe_fused_down_fp8_op(int64_t ptr, const at::Tensor& h, const at::Tensor& h_scale,
                           const at::Tensor& w2, const at::Tensor& w2_scale,
                           const std::optional<at::Tensor>& status) {
  AllToAll* ata = lookup(ptr);
  const FusedFfnFp8Call f = make_fp8_ffn_call(*ata, w2, w2_scale, h, h_scale, false, status);
  const c10::cuda::OptionalCUDAGuard guard(h.device());
  guarded([&] { ata->fused_down_fp8(f, at::cuda::getCurrentCUDAStream()); });
}

void fake_moe_fused_up_fp8(int64_t, const at::Tensor&, const at::Tensor&, at::Tensor&, at::Tensor&,
                           const std::optional<at::Tensor>&, const std::optional<at::Tensor>&) {}
void fake_moe_fused_down_fp8(int64_t, const at::Tensor&, const at::Tensor&, const at::Tensor&,
                             const at::Tensor&, const std::optional<at::Tensor>&) {}

void fake_moe_fused_up(int64_t, const at::Tensor&, at::Tensor&, const std::optional<at::Tensor>&,
                       const std::optional<at::Tensor>&, int64_t) {}
void fake_moe_fused_down(int64_t, const at::Tensor&, const at::Tensor&,
                         const std::optional<at::Tensor>&, int64_t) {}

void set_trace_op(int64_t ptr, bool on) { lookup(ptr)->set_trace(on); }

std::vector<int64_t> read_trace_op(int64_t ptr) {
  const std::vector<uint64_t> t = guarded([&] { return lookup(ptr)->read_trace(); });
  return std::vector<int64_t>(t.begin(), t.end());
}

std::vector<int64_t> layout_op(int64_t ptr) {
  const A2AParams& p = lookup(ptr)->params();
  return {p.nle, p.num_dp_groups, p.cap, p.region_slots, p.slot_bytes,
          static_cast<int64_t>(p.arena_bytes), p.ll, p.ll_slot_bytes, p.ll_comb_slot_bytes,
          p.tiny, lookup(ptr)->arena().from_vmm() ? 1 : 0, p.mc != nullptr ? 1 : 0};
}

std::string multicast_note_op(int64_t ptr) { return lookup(ptr)->arena().multicast_note();
}

// -------------------------------------------------------- symmetric memory ----

at::Tensor get_unique_id() {
  const UniqueId id = guarded([] { return create_unique_id(); });
  at::Tensor t = at::empty({static_cast<int64_t>(kUniqueIdBytes)},
                           at::TensorOptions().dtype(at::kByte).device(at::kCPU));
  std::memcpy(t.data_ptr(), id.bytes, kUniqueIdBytes);
  return t;
}

int64_t unique_id_size() { return static_cast<int64_t>(kUniqueIdBytes); }

int64_t init_op(const at::Tensor& uid, int64_t rank, int64_t world_size) {
  TORCH_CHECK(uid.device().is_cpu() && uid.scalar_type() == at::kByte && uid.is_contiguous() &&
                  uid.numel() == static_cast<int64_t>(kUniqueIdBytes),
              "uid must be a contiguous CPU uint8 tensor of ", kUniqueIdBytes, " bytes");
  guarded([&] {
    UniqueId id{};
    std::memcpy(id.bytes, uid.data_ptr(), kUniqueIdBytes);
    Runtime::instance().init(std::make_shared<SocketBootstrap>(
        id, static_cast<int>(rank), static_cast<int>(world_size),
        static_cast<int>(env_long("PPLX_B200_BOOTSTRAP_TIMEOUT_MS", 60000))));
  });
  return 0;
}

void finalize_op() {
  guarded([] { Runtime::instance().finalize(); });
}

int64_t my_pe_op() {
  return guarded([] { return static_cast<int64_t>(Runtime::instance().my_pe()); });
}

int64_t n_pes_op() {
  return guarded([] { return static_cast<int64_t>(Runtime::instance().n_pes()); });
}

at::Tensor malloc_op(const std::vector<int64_t>& shape, c10::ScalarType dtype,
                     const c10::Device& device) {
  TORCH_CHECK(device.is_cuda(), "symmetric memory lives on CUDA devices");
  const c10::cuda::OptionalCUDAGuard guard(device);
  int64_t numel = 1;
  for (int64_t d : shape) numel *= d;
  const size_t bytes = static_cast<size_t>(numel) * c10::elementSize(dtype);
  auto alloc = guarded([&] { return Runtime::instance().malloc(bytes); });
  void* ptr = alloc->local();
  return at::from_blob(
      ptr, shape, [ptr](void*) { Runtime::instance().release(ptr); },
      at::TensorOptions().dtype(dtype).device(at::kCUDA, current_device()));
}

void barrier_all_op() {
  guarded([] { Runtime::instance().barrier_all(); });
}

void barrier_all_on_current_stream_op() {
  guarded([] { Runtime::instance().barrier_on_stream(at::cuda::getCurrentCUDAStream()); });
}

void alltoall_op(at::Tensor& dest, const at::Tensor& source) {
  TORCH_CHECK(dest.is_cuda() && source.is_cuda() && dest.is_contiguous() &&
                  source.is_contiguous() && dest.nbytes() == source.nbytes(),
              "alltoall: dest and source must be contiguous CUDA tensors of equal size");
  TORCH_CHECK(dest.dim() >= 1 && dest.size(0) == Runtime::instance().n_pes(),
              "alltoall: dest.size(0) must equal the number of ranks");
  const c10::cuda::OptionalCUDAGuard guard(dest.device());
  guarded([&] {
    Runtime::instance().alltoall(dest.data_ptr(), source.data_ptr(), dest.nbytes() / dest.size(0),
                                 at::cuda::getCurrentCUDAStream());
  });
}

void fake_alltoall(at::Tensor&, const at::Tensor&) {}

// ----------------------------------------------------------------- utils ----

// Host-only exercise of the socket bootstrap: gathers one word per rank and runs
// an all-to-all of (source, destination) pairs.  Returns [world + world] int64.
at::Tensor bootstrap_selftest_op(const at::Tensor& uid, int64_t rank, int64_t world_size,
                                 int64_t timeout_ms) {
  TORCH_CHECK(uid.device().is_cpu() && uid.scalar_type() == at::kByte &&
                  uid.numel() == static_cast<int64_t>(kUniqueIdBytes),
              "uid must be a CPU uint8 tensor of ", kUniqueIdBytes, " bytes");
  return guarded([&] {
    UniqueId id{};
    std::memcpy(id.bytes, uid.contiguous().data_ptr(), kUniqueIdBytes);
    SocketBootstrap bs(id, static_cast<int>(rank), static_cast<int>(world_size),
                       static_cast<int>(timeout_ms));
    const int64_t w = world_size;
    at::Tensor out = at::zeros({2 * w}, at::TensorOptions().dtype(at::kLong));
    int64_t* o = out.data_ptr<int64_t>();
    const int64_t mine = 1000 + rank;
    bs.all_gather(&mine, o, sizeof(int64_t));
    std::vector<int64_t> send(w);
    for (int64_t d = 0; d < w; ++d) send[d] = rank * 100 + d;
    bs.all_to_all(send.data(), o + w, sizeof(int64_t));
    bs.barrier();
    return out;
  });
}

// Host-only exercise of the descriptor exchange that the VMM arena uses: every rank puts a
// word into an anonymous file and passes the descriptor to all peers (the last rank of a
// world of three or more passes none); returns what was read through the received
// descriptors, -1 where none came, -2 at the caller's own index.
at::Tensor fd_exchange_selftest_op(const at::Tensor& uid, int64_t rank, int64_t world_size,
                                   int64_t timeout_ms) {
  TORCH_CHECK(uid.device().is_cpu() && uid.scalar_type() == at::kByte &&
                  uid.numel() == static_cast<int64_t>(kUniqueIdBytes),
              "uid must be a CPU uint8 tensor of ", kUniqueIdBytes, " bytes");
  return guarded([&] {
    UniqueId id{};
    std::memcpy(id.bytes, uid.contiguous().data_ptr(), kUniqueIdBytes);
    SocketBootstrap bs(id, static_cast<int>(rank), static_cast<int>(world_size),
                       static_cast<int>(timeout_ms));
    int mine = -1;
    if (!(world_size >= 3 && rank == world_size - 1)) {
      mine = ::memfd_create("pplx-fd-selftest", MFD_CLOEXEC);
      PPLX_CHECK(mine >= 0, "memfd_create failed");
      const int64_t word = 7000 + rank;
      PPLX_CHECK(::pwrite(mine, &word, sizeof(word), 0) == sizeof(word), "pwrite failed");
    }
    const std::vector<int> fds = exchange_fds(bs, mine, static_cast<int>(timeout_ms));
    if (mine >= 0) ::close(mine);
    at::Tensor out = at::full({world_size}, -1, at::TensorOptions().dtype(at::kLong));
    int64_t* o = out.data_ptr<int64_t>();
    o[rank] = -2;
    for (int64_t r = 0; r < world_size; ++r) {
      if (fds[r] < 0) continue;
      int64_t word = 0;
      PPLX_CHECK(::pread(fds[r], &word, sizeof(word), 0) == sizeof(word), "pread failed");
      o[r] = word;
      ::close(fds[r]);
    }
    return out;
  });
}

void sleep_on_stream_op(double seconds) {
  CUDA_CHECK(launch_sleep(static_cast<uint64_t>(seconds * 1e9), at::cuda::getCurrentCUDAStream()));
}

std::vector<int64_t> wait_probe_op(const at::Tensor& flag, double timeout_ms) {
  TORCH_CHECK(flag.is_cuda() && flag.element_size() == 4 && flag.numel() >= 1,
              "flag must be a 32-bit CUDA tensor");
  const c10::cuda::OptionalCUDAGuard guard(flag.device());
  return guarded([&] {
    DeviceBuffer<Status> st(1);
    auto stream = at::cuda::getCurrentCUDAStream();
    CUDA_CHECK(launch_wait_probe(static_cast<const uint32_t*>(flag.data_ptr()), st.get(),
                                 static_cast<uint64_t>(timeout_ms * 1e6), stream));
    CUDA_CHECK(cudaStreamSynchronize(stream));
    const Status s = st.to_host()[0];
    return std::vector<int64_t>{s.code, s.phase, s.peer, s.expected, s.observed};
  });
}

}  // namespace

void register_all_to_all_ops(torch::Library& m) {
  m.def("all_to_all_intranode_create(int max_num_tokens, int num_experts, int experts_per_token, "
        "int rank, int world_size, int dp_size, int hidden_dim, int hidden_dim_bytes, "
        "int hidden_dim_scale_bytes, str group_name) -> int",
        &create_intranode);
  m.def("all_to_all_internode_create(int max_num_tokens, int num_experts, int experts_per_token, "
        "int rank, int world_size, int dp_size, int hidden_dim, int hidden_dim_bytes, "
        "int hidden_dim_scale_bytes) -> int",
        &create_internode);
  m.def("all_to_all_local_world_create(int max_num_tokens, int num_experts, "
        "int experts_per_token, int world_size, int dp_size, int hidden_dim, "
        "int hidden_dim_bytes, int hidden_dim_scale_bytes) -> int[]",
        &create_local_world);
  m.def("all_to_all_destroy(int ptr) -> ()", &destroy);

  const char* dispatch_args =
      "(int ptr, Tensor! out_expert_num_tokens, Tensor! out_expert_x, "
      "Tensor!? out_expert_x_scale, Tensor dp_x, Tensor? dp_x_scale, Tensor indices, "
      "Tensor? bound_m, bool do_send, bool do_recv) -> ()";
  const char* combine_args =
      "(int ptr, Tensor! out_tokens, Tensor indices, Tensor weights, Tensor expert_y, "
      "Tensor? bound_m, bool do_send, bool do_recv) -> ()";
  for (const char* flavour : {"intranode", "internode"}) {
    const std::string d = std::string("all_to_all_") + flavour + "_dispatch";
    const std::string c = std::string("all_to_all_") + flavour + "_combine";
    m.def((d + dispatch_args).c_str());
    m.impl(d.c_str(), c10::kCUDA, &dispatch_op);
    m.impl(d.c_str(), c10::kMeta, &fake_dispatch);
    m.def((c + combine_args).c_str());
    m.impl(c.c_str(), c10::kCUDA, &combine_op);
    m.impl(c.c_str(), c10::kMeta, &fake_combine);
  }

  m.def("all_to_all_dispatch_quant(int ptr, Tensor! out_expert_num_tokens, Tensor! out_expert_x, "
        "Tensor! out_expert_x_scale, Tensor dp_x, Tensor indices, Tensor? bound_m, bool do_send, "
        "bool do_recv) -> ()");
  m.impl("all_to_all_dispatch_quant", c10::kCUDA, &dispatch_quant_op);
  m.impl("all_to_all_dispatch_quant", c10::kMeta, &fake_dispatch_quant);
  m.def("all_to_all_dispatch_group(int[] ptrs, Tensor[] out_expert_num_tokens, "
        "Tensor[] out_expert_x, Tensor[] out_expert_x_scale, Tensor[] dp_x, Tensor[] dp_x_scale, "
        "Tensor[] indices, Tensor[] bound_m, bool do_send, bool do_recv) -> ()",
        &dispatch_group_op);
  m.def("all_to_all_dispatch_quant_group(int[] ptrs, Tensor[] out_expert_num_tokens, "
        "Tensor[] out_expert_x, Tensor[] out_expert_x_scale, Tensor[] dp_x, Tensor[] indices, "
        "Tensor[] bound_m) -> ()",
        &dispatch_quant_group_op);
  m.def("all_to_all_combine_group(int[] ptrs, Tensor[] out_tokens, Tensor[] indices, "
        "Tensor[] weights, Tensor[] expert_y, Tensor[] bound_m, bool do_send, bool do_recv) -> ()",
        &combine_group_op);

  m.def("all_to_all_status(int ptr) -> int[]", &status_op);
  m.def("all_to_all_check_status(int ptr) -> ()", &check_status_op);
  m.def("all_to_all_peek_status(int ptr) -> int[]", &peek_status_op);
  m.def("all_to_all_reset(int ptr) -> ()", &reset_op);
  m.def("all_to_all_verify_canaries(int ptr) -> ()", &verify_canaries_op);
  m.def("all_to_all_set_timeout_ms(int ptr, float ms) -> ()", &set_timeout_ms_op);
  m.def("all_to_all_set_debug_checks(int ptr, bool on) -> ()", &set_debug_checks_op);
  m.def("all_to_all_set_quant_pow2(int ptr, bool on) -> ()", &set_quant_pow2_op);
  m.def("all_to_all_set_max_blocks(int ptr, int n) -> ()", &set_max_blocks_op);
  m.def("all_to_all_layout(int ptr) -> int[]", &layout_op);
  m.def("all_to_all_multicast_note(int ptr) -> str", &multicast_note_op);
  m.def("all_to_all_set_trace(int ptr, bool on) -> ()", &set_trace_op);
  m.def("all_to_all_set_combine_units(int ptr, int units) -> ()", &set_combine_units_op);
  m.def("moe_dispatch_send(int ptr, Tensor dp_x, Tensor indices, Tensor? bound_m, "
        "bool quantize=False) -> ()");
  m.impl("moe_dispatch_send", c10::kCUDA, &moe_dispatch_send_op);
  m.impl("moe_dispatch_send", c10::kMeta, &fake_moe_dispatch_send);
  m.def("moe_dispatch_send_group(int[] ptrs, Tensor[] dp_x, Tensor[] indices, "
        "Tensor[] bound_m, bool quantize=False) -> ()",
        &moe_dispatch_send_group_op);
  m.def("moe_fused_up_fp8(int ptr, Tensor w13, Tensor w13_scale, Tensor! h, Tensor! h_scale, "
        "Tensor!? out_expert_num_tokens, Tensor!? status) -> ()");
  m.impl("moe_fused_up_fp8", c10::kCUDA, &moe_fused_up_fp8_op);
  m.impl("moe_fused_up_fp8", c10::kMeta, &fake_moe_fused_up_fp8);
  m.def("moe_fused_down_fp8(int ptr, Tensor h, Tensor h_scale, Tensor w2, Tensor w2_scale, "
        "Tensor!? status) -> ()");
  m.impl("moe_fused_down_fp8", c10::kCUDA, &moe_fused_down_fp8_op);
  m.impl("moe_fused_down_fp8", c10::kMeta, &fake_moe_fused_down_fp8);
  m.def("moe_fused_up(int ptr, Tensor w13, Tensor! h, Tensor!? out_expert_num_tokens, "
        "Tensor!? status, int expected_rows=0) -> ()");
  m.impl("moe_fused_up", c10::kCUDA, &moe_fused_up_op);
  m.impl("moe_fused_up", c10::kMeta, &fake_moe_fused_up);
  m.def("moe_fused_down(int ptr, Tensor h, Tensor w2, Tensor!? status, "
        "int expected_rows=0) -> ()");
  m.impl("moe_fused_down", c10::kCUDA, &moe_fused_down_op);
  m.impl("moe_fused_down", c10::kMeta, &fake_moe_fused_down);
  m.def("all_to_all_read_trace(int ptr) -> int[]", &read_trace_op);
}

void register_symmetric_memory_ops(torch::Library& m) {
  m.def("nvshmem_get_unique_id", &get_unique_id);
  m.def("nvshmem_unique_id_size", &unique_id_size);
  m.def("nvshmem_init", &init_op);
  m.def("nvshmem_finalize", &finalize_op);
  m.def("nvshmem_my_pe", &my_pe_op);
  m.def("nvshmem_n_pes", &n_pes_op);
  m.def("nvshmem_malloc", &malloc_op);
  m.def("nvshmem_barrier_all", &barrier_all_op);
  m.def("nvshmem_barrier_all_on_current_stream", &barrier_all_on_current_stream_op);
  m.def("nvshmem_alltoall(Tensor! dest, Tensor src) -> ()");
  m.impl("nvshmem_alltoall", c10::kCUDA, &alltoall_op);
  m.impl("nvshmem_alltoall", c10::kMeta, &fake_alltoall);

  m.def("bootstrap_selftest(Tensor uid, int rank, int world_size, int timeout_ms) -> Tensor",
        &bootstrap_selftest_op);
  m.def("fd_exchange_selftest(Tensor uid, int rank, int world_size, int timeout_ms) -> Tensor",
        &fd_exchange_selftest_op);
  m.def("sleep_on_stream(float seconds) -> ()", &sleep_on_stream_op);
  m.def("wait_probe(Tensor flag, float timeout_ms) -> int[]", &wait_probe_op);
}

}  // namespace pplx

TORCH_LIBRARY(pplx_kernels_b200, m) {
  pplx::register_all_to_all_ops(m);
  pplx::register_symmetric_memory_ops(m);
  pplx::register_extension_ops(m);
}

PPLX_REGISTER_EXTENSION(libpplx_kernels_b200)
