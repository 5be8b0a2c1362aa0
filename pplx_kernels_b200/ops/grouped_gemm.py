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
