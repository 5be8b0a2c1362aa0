// Operators that have no counterpart in the reference: the tcgen05 grouped
// expert GEMM (and, built on it, the pieces of the fused MoE layer).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "../core/utils.h"
#include "../kernels/grouped_gemm.h"
#include "registration.h"

namespace pplx {
namespace {

// out[e, :counts[e]] = act(x[e, :counts[e]] @ w[e]^T), bf16 in / bf16 out.
void grouped_gemm_op(const at::Tensor& x, const at::Tensor& w, const at::Tensor& counts,
                     at::Tensor& out, bool swiglu, const std::optional<at::Tensor>& status,
                     int64_t expected_rows, int64_t half_n, int64_t cta_pair) {
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && counts.is_cuda() && out.is_cuda(),
              "grouped_gemm: all tensors must be CUDA tensors");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 &&
                  out.scalar_type() == at::kBFloat16,
              "grouped_gemm: x, w and out must be bfloat16");
  TORCH_CHECK(x.dim() == 3 && w.dim() == 3 && out.dim() == 3, "grouped_gemm: 3-D tensors expected");
  TORCH_CHECK(x.stride(2) == 1 && w.stride(2) == 1 && out.stride(2) == 1,
              "grouped_gemm: the last dimension must be contiguous");
  const int64_t E = x.size(0), rows = x.size(1), K = x.size(2);
  const int64_t n_out = out.size(2);
  TORCH_CHECK(w.size(0) == E && w.size(2) == K && w.size(1) == (swiglu ? 2 * n_out : n_out),
              "grouped_gemm: w must be [experts, ", swiglu ? "2 * " : "", "n_out, k]");
  TORCH_CHECK(out.size(0) == E && out.size(1) == rows, "grouped_gemm: out must be [experts, rows, n_out]");
  TORCH_CHECK(counts.scalar_type() == at::kInt && counts.numel() == E && counts.is_contiguous(),
              "grouped_gemm: counts must be a contiguous int32 tensor of [experts]");
  uint32_t* status_ptr = nullptr;
  if (status.has_value()) {
    TORCH_CHECK(status->is_cuda() && status->element_size() == 4 && status->numel() >= 1,
                "grouped_gemm: status must be a 32-bit CUDA tensor");
    status_ptr = static_cast<uint32_t*>(status->data_ptr());
  }
  const c10::cuda::OptionalCUDAGuard guard(x.device());
  GroupedGemmCall c;
  c.x = x.data_ptr();
  c.x_stride_e = x.stride(0);
  c.x_stride_row = x.stride(1);
  c.w = w.data_ptr();
  c.w_stride_e = w.stride(0);
  c.w_stride_row = w.stride(1);
  c.counts = counts.data_ptr<int32_t>();
  c.out = out.data_ptr();
  c.out_stride_e = out.stride(0);
  c.out_stride_row = out.stride(1);
  c.status = status_ptr;
  c.num_experts = static_cast<int>(E);
  c.rows_per_expert = static_cast<int>(rows);
  c.n_out = static_cast<int>(n_out);
  c.k = static_cast<int>(K);
  c.swiglu = swiglu;
  c.expected_total_rows = expected_rows;
  c.half_n = static_cast<int>(half_n);
  c.cta_pair = static_cast<int>(cta_pair);
  try {
    launch_grouped_gemm(c, at::cuda::getCurrentCUDAStream());
  } catch (const Error& e) {
    TORCH_CHECK(false, e.what());
  }
}

void fake_grouped_gemm(const at::Tensor&, const at::Tensor&, const at::Tensor&, at::Tensor&, bool,
                       const std::optional<at::Tensor>&, int64_t, int64_t, int64_t) {}

}  // namespace

void register_extension_ops(torch::Library& m) {
  m.def("grouped_gemm(Tensor x, Tensor w, Tensor counts, Tensor! out, bool swiglu, "
        "Tensor!? status, int expected_rows=0, int half_n=0, int cta_pair=-1) -> ()");
  m.impl("grouped_gemm", c10::kCUDA, &grouped_gemm_op);
  m.impl("grouped_gemm", c10::kMeta, &fake_grouped_gemm);
}

}  // namespace pplx
