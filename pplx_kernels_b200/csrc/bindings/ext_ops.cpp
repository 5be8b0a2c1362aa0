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

// Block-scaled fp8 grouped GEMM: e4m3 operands, fp32 scale per row x 128 columns (x) and per
// 128 x 128 block (w).
void grouped_gemm_fp8_op(const at::Tensor& xq, const at::Tensor& sa, const at::Tensor& wq,
                         const at::Tensor& sw, const at::Tensor& counts, at::Tensor& out,
                         const std::optional<at::Tensor>& out_scale, bool swiglu_quant,
                         const std::optional<at::Tensor>& status, bool pow2_scales) {
  TORCH_CHECK(xq.is_cuda() && wq.is_cuda() && sa.is_cuda() && sw.is_cuda() && out.is_cuda(),
              "grouped_gemm_fp8: all tensors must be CUDA tensors");
  TORCH_CHECK(xq.element_size() == 1 && wq.element_size() == 1, "xq and wq must be 1-byte (e4m3)");
  TORCH_CHECK(xq.dim() == 3 && wq.dim() == 3 && out.dim() == 3 && sa.dim() == 3 && sw.dim() == 3,
              "grouped_gemm_fp8: 3-D tensors expected");
  TORCH_CHECK(xq.stride(2) == 1 && wq.stride(2) == 1 && out.stride(2) == 1 && sa.stride(2) == 1 &&
                  sw.stride(2) == 1,
              "grouped_gemm_fp8: the last dimension must be contiguous");
  TORCH_CHECK(sa.scalar_type() == at::kFloat && sw.scalar_type() == at::kFloat,
              "scales must be float32");
  const int64_t E = xq.size(0), rows = xq.size(1), K = xq.size(2);
  const int64_t n_out = out.size(2);
  const int64_t kb = (K + 127) / 128;
  const int64_t w_rows = swiglu_quant ? 2 * n_out : n_out;
  TORCH_CHECK(wq.size(0) == E && wq.size(1) == w_rows && wq.size(2) == K, "wq has the wrong shape");
  TORCH_CHECK(sa.size(0) == E && sa.size(1) == rows && sa.size(2) == kb, "sa must be [E, rows, K/128]");
  TORCH_CHECK(sw.size(0) == E && sw.size(1) == (w_rows + 127) / 128 && sw.size(2) == kb,
              "sw must be [E, ceil(w rows / 128), K/128]");
  TORCH_CHECK(out.size(0) == E && out.size(1) == rows, "out must be [E, rows, n_out]");
  TORCH_CHECK(counts.scalar_type() == at::kInt && counts.numel() == E && counts.is_contiguous(),
              "counts must be a contiguous int32 tensor of [E]");
  Fp8GemmCall c;
  if (swiglu_quant) {
    TORCH_CHECK(out.element_size() == 1, "with swiglu_quant the output is e4m3");
    TORCH_CHECK(out_scale.has_value() && out_scale->is_cuda() && out_scale->dim() == 3 &&
                    out_scale->scalar_type() == at::kFloat && out_scale->stride(2) == 1 &&
                    out_scale->size(0) == E && out_scale->size(1) == rows &&
                    out_scale->size(2) == n_out / 128,
                "out_scale must be float32 [E, rows, n_out / 128]");
    c.out_scale = out_scale->data_ptr<float>();
    c.os_stride_e = out_scale->stride(0);
    c.os_stride_row = out_scale->stride(1);
  } else {
    TORCH_CHECK(out.scalar_type() == at::kBFloat16, "the plain epilogue writes bfloat16");
  }
  if (status.has_value()) {
    TORCH_CHECK(status->is_cuda() && status->element_size() == 4, "status must be a 32-bit CUDA tensor");
    c.status = static_cast<uint32_t*>(status->data_ptr());
  }
  const c10::cuda::OptionalCUDAGuard guard(xq.device());
  c.x = xq.data_ptr();
  c.x_stride_e = xq.stride(0);
  c.x_stride_row = xq.stride(1);
  c.sa = sa.data_ptr<float>();
  c.sa_stride_e = sa.stride(0);
  c.sa_stride_row = sa.stride(1);
  c.w = wq.data_ptr();
  c.w_stride_e = wq.stride(0);
  c.w_stride_row = wq.stride(1);
  c.sw = sw.data_ptr<float>();
  c.sw_stride_e = sw.stride(0);
  c.sw_stride_row = sw.stride(1);
  c.counts = counts.data_ptr<int32_t>();
  c.out = out.data_ptr();
  c.out_stride_e = out.stride(0);
  c.out_stride_row = out.stride(1);
  c.num_experts = static_cast<int>(E);
  c.rows_per_expert = static_cast<int>(rows);
  c.n_out = static_cast<int>(n_out);
  c.k = static_cast<int>(K);
  c.swiglu_quant = swiglu_quant;
  c.pow2_scales = pow2_scales;
  try {
    launch_grouped_gemm_fp8(c, at::cuda::getCurrentCUDAStream());
  } catch (const Error& e) {
    TORCH_CHECK(false, e.what());
  }
}

void fake_grouped_gemm_fp8(const at::Tensor&, const at::Tensor&, const at::Tensor&,
                           const at::Tensor&, const at::Tensor&, at::Tensor&,
                           const std::optional<at::Tensor>&, bool,
                           const std::optional<at::Tensor>&, bool) {}

}  // namespace

void register_extension_ops(torch::Library& m) {
  m.def("grouped_gemm(Tensor x, Tensor w, Tensor counts, Tensor! out, bool swiglu, "
        "Tensor!? status, int expected_rows=0, int half_n=0, int cta_pair=-1) -> ()");
  m.impl("grouped_gemm", c10::kCUDA, &grouped_gemm_op);
  m.impl("grouped_gemm", c10::kMeta, &fake_grouped_gemm);
  m.def("grouped_gemm_fp8(Tensor xq, Tensor sa, Tensor wq, Tensor sw, Tensor counts, Tensor! out, "
        "Tensor!? out_scale, bool swiglu_quant, Tensor!? status, bool pow2_scales=False) -> ()");
  m.impl("grouped_gemm_fp8", c10::kCUDA, &grouped_gemm_fp8_op);
  m.impl("grouped_gemm_fp8", c10::kMeta, &fake_grouped_gemm_fp8);
}

}  // namespace pplx
