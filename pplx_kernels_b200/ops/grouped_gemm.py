"""Grouped expert GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory + TMA).

``grouped_gemm(x, w, counts)`` computes, for every expert ``e``,
``out[e, :counts[e]] = x[e, :counts[e]] @ w[e].T`` in bf16 with fp32 accumulation;
with ``swiglu=True`` the weight stacks a gate and an up projection
(``w[e]`` is ``[2 * I, K]``, gate rows first) and the result is
``silu(x @ gate.T) * (x @ up.T)`` with ``I`` columns.  Rows at or beyond
``counts[e]`` are left untouched.  The reference library has no GEMM; this is
part of the fused MoE path that goes beyond it.
"""

from __future__ import annotations

import torch

from . import _ops


def grouped_gemm(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor,
                 out: torch.Tensor | None = None, swiglu: bool = False,
                 status: torch.Tensor | None = None, expected_rows: int = 0,
                 half_n: int = 0, cta_pair: int = -1) -> torch.Tensor:
    """x: [E, rows, K] bf16, w: [E, N or 2N, K] bf16, counts: [E] int32 -> out [E, rows, N] bf16.

    ``expected_rows`` (total valid rows, 0 = capacity) and ``half_n`` (0 = choose) steer the
    tile width: the accumulator is ``2 * half_n`` columns wide and the launcher picks the
    width that fills the last wave of tiles best.  ``cta_pair`` selects the kernel form:
    1 = two CTAs share a 256-row tile (tcgen05 ``cta_group::2``, less shared-memory traffic
    per flop), 0 = one CTA per 128-row tile, -1 = choose from the expected rows per expert.
    """
    n_out = w.size(1) // 2 if swiglu else w.size(1)
    if out is None:
        out = torch.empty(x.size(0), x.size(1), n_out, dtype=torch.bfloat16, device=x.device)
    _ops.grouped_gemm(x, w, counts, out, swiglu, status, expected_rows, half_n, cta_pair)
    return out


def grouped_gemm_reference(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor,
                           swiglu: bool = False) -> torch.Tensor:
    """Plain PyTorch fp32 statement of the same operation (rows beyond counts are zero)."""
    E, rows, _ = x.shape
    n_out = w.size(1) // 2 if swiglu else w.size(1)
    out = torch.zeros(E, rows, n_out, dtype=torch.float32, device=x.device)
    for e, m in enumerate(counts.tolist()):
        if m == 0:
            continue
        y = x[e, :m].to(torch.float32) @ w[e].to(torch.float32).t()
        if swiglu:
            gate, up = y[:, :n_out], y[:, n_out:]
            y = torch.nn.functional.silu(gate) * up
        out[e, :m] = y
    return out


def grouped_gemm_fp8(xq: torch.Tensor, sa: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor,
                     counts: torch.Tensor, swiglu_quant: bool = False,
                     out: torch.Tensor | None = None, out_scale: torch.Tensor | None = None,
                     status: torch.Tensor | None = None, pow2_scales: bool = False):
    """Block-scaled fp8 grouped GEMM (tcgen05 ``kind::f8f6f4``, or with ``pow2_scales``
    ``kind::mxf8f6f4.block_scale``).

    ``xq`` [E, rows, K] and ``wq`` [E, N (or 2N), K] are ``float8_e4m3fn``; ``sa`` [E, rows,
    K/128] holds one fp32 scale per row and 128 columns, ``sw`` [E, ceil(w rows/128), K/128]
    one per 128 x 128 block of the weight.  Plain: returns bf16 [E, rows, N].  With
    ``swiglu_quant`` (``wq`` stacks gate and up rows): returns ``(hq, hs)`` -- silu(gate) * up
    quantised to e4m3 with one fp32 scale per row and 128 columns, the input format of the
    next GEMM.

    ``pow2_scales=True`` is the caller's promise that every scale in ``sa`` and ``sw`` is a power
    of two (``per_token_block_quant(..., pow2=True)``, ``quantize_weight_blocks(..., pow2=True)``,
    ``dispatch_quant(..., pow2=True)``): the tensor cores then apply the scales themselves and the
    whole K range accumulates in tensor memory; the ``swiglu_quant`` epilogue emits power-of-two
    scales in turn.  Mantissa bits of a scale that is not a power of two would be ignored.
    """
    E, rows, _ = xq.shape
    n_out = wq.size(1) // 2 if swiglu_quant else wq.size(1)
    if swiglu_quant:
        if out is None:
            out = torch.empty(E, rows, n_out, dtype=torch.float8_e4m3fn, device=xq.device)
        if out_scale is None:
            out_scale = torch.empty(E, rows, n_out // 128, dtype=torch.float32, device=xq.device)
    elif out is None:
        out = torch.empty(E, rows, n_out, dtype=torch.bfloat16, device=xq.device)
    _ops.grouped_gemm_fp8(xq, sa, wq, sw, counts, out, out_scale, swiglu_quant, status,
                          pow2_scales)
    return (out, out_scale) if swiglu_quant else out


def quantize_weight_blocks(w: torch.Tensor, block: int = 128,
                           pow2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """w: [E, N, K] -> (e4m3 [E, N, K], fp32 scales [E, ceil(N/block), ceil(K/block)]).
    With ``pow2`` every scale is rounded up to a power of two (hardware block scaling)."""
    E, N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wf = torch.nn.functional.pad(w.to(torch.float32), (0, kb * block - K, 0, nb * block - N))
    v = wf.view(E, nb, block, kb, block)
    scale = v.abs().amax(dim=(2, 4)).clamp(min=1e-4) / 448.0
    if pow2:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (v / scale[:, :, None, :, None]).clamp(-448.0, 448.0)
    q = q.view(E, nb * block, kb * block)[:, :N, :K].to(torch.float8_e4m3fn).contiguous()
    return q, scale.contiguous()


def grouped_gemm_fp8_reference(xq: torch.Tensor, sa: torch.Tensor, wq: torch.Tensor,
                               sw: torch.Tensor, counts: torch.Tensor,
                               swiglu: bool = False) -> torch.Tensor:
    """Plain PyTorch fp32 statement: dequantise both operands, multiply, optional SwiGLU."""
    E, rows, K = xq.shape
    x = xq.to(torch.float32) * sa.repeat_interleave(128, dim=2)[:, :, :K]
    w = wq.to(torch.float32) * sw.repeat_interleave(128, dim=1)[:, : wq.size(1)].repeat_interleave(
        128, dim=2)[:, :, :K]
    n_out = wq.size(1) // 2 if swiglu else wq.size(1)
    out = torch.zeros(E, rows, n_out, dtype=torch.float32, device=xq.device)
    for e, m in enumerate(counts.tolist()):
        if m == 0:
            continue
        y = x[e, :m] @ w[e].t()
        if swiglu:
            y = torch.nn.functional.silu(y[:, :n_out]) * y[:, n_out:]
        out[e, :m] = y
    return out
