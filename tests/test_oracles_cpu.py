"""CPU tests of the plain-PyTorch oracles that the GPU numerics tests compare against
(block quantisation, grouped GEMM references, the MoE layer reference)."""

import torch

from pplx_kernels_b200.models.moe import moe_reference
from pplx_kernels_b200.ops.grouped_gemm import (
    grouped_gemm_fp8_reference,
    grouped_gemm_reference,
    quantize_weight_blocks,
)
from pplx_kernels_b200.ops.quant import block_dequant, per_token_block_quant


def test_block_quantisation_round_trip_and_scale_rule():
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(7, 300, generator=gen) * 3
    x[2] = 0  # an all-zero row keeps the scale floor
    q, s = per_token_block_quant(x)
    assert q.dtype == torch.float8_e4m3fn and q.shape == x.shape and s.shape == (7, 3)
    # scale = max(amax, 1e-4) / 448 per row and 128 columns (the last block is ragged)
    amax = torch.stack([x[:, :128].abs().amax(1), x[:, 128:256].abs().amax(1),
                        x[:, 256:].abs().amax(1)], dim=1).clamp(min=1e-4)
    torch.testing.assert_close(s, amax / 448.0)
    back = block_dequant(q, s)
    # e4m3 keeps 3 mantissa bits: the error is within 1/16 of the block maximum
    assert ((back - x).abs() <= amax.repeat_interleave(128, dim=1)[:, :300] / 16 + 1e-6).all()
    assert (back[2] == 0).all()


def test_weight_block_quantisation_shapes_and_error():
    gen = torch.Generator().manual_seed(1)
    w = torch.randn(2, 200, 260, generator=gen)
    q, s = quantize_weight_blocks(w)
    assert q.shape == w.shape and q.dtype == torch.float8_e4m3fn and s.shape == (2, 2, 3)
    deq = q.float() * s.repeat_interleave(128, dim=1)[:, :200].repeat_interleave(128, dim=2)[..., :260]
    assert (deq - w).abs().max() <= w.abs().max() / 16 + 1e-6


def test_grouped_gemm_references_agree_with_dense_math():
    gen = torch.Generator().manual_seed(2)
    E, rows, K, N = 3, 10, 256, 128
    x = torch.randn(E, rows, K, generator=gen)
    w = torch.randn(E, 2 * N, K, generator=gen) * K ** -0.5
    counts = torch.tensor([10, 0, 4], dtype=torch.int32)
    out = grouped_gemm_reference(x.bfloat16(), w.bfloat16(), counts, swiglu=True)
    for e, m in enumerate(counts.tolist()):
        h = x[e, :m].bfloat16().float() @ w[e].bfloat16().float().t()
        want = torch.nn.functional.silu(h[:, :N]) * h[:, N:]
        torch.testing.assert_close(out[e, :m].float(), want, rtol=2e-2, atol=2e-2)

    # the fp8 reference is the same contraction over de-quantised operands
    xq, sa = per_token_block_quant(x.view(E * rows, K))
    wq, sw = quantize_weight_blocks(w[:, :N])
    got = grouped_gemm_fp8_reference(xq.view(E, rows, K), sa.view(E, rows, -1), wq, sw, counts)
    xd = block_dequant(xq, sa).view(E, rows, K)
    wd = wq.float() * sw.repeat_interleave(128, dim=1)[:, :N].repeat_interleave(128, dim=2)[..., :K]
    for e, m in enumerate(counts.tolist()):
        torch.testing.assert_close(got[e, :m], xd[e, :m] @ wd[e].t(), rtol=1e-4, atol=1e-4)


def test_moe_reference_is_the_weighted_sum_of_expert_ffns():
    gen = torch.Generator().manual_seed(3)
    E, H, inter, m, topk = 4, 32, 16, 6, 2
    x = torch.randn(m, H, generator=gen).bfloat16()
    w13 = (torch.randn(E, 2 * inter, H, generator=gen) * 0.2).bfloat16()
    w2 = (torch.randn(E, H, inter, generator=gen) * 0.2).bfloat16()
    idx = torch.stack([torch.randperm(E, generator=gen)[:topk] for _ in range(m)])
    wts = torch.softmax(torch.randn(m, topk, generator=gen), dim=-1)
    out = moe_reference(x, idx, wts, w13, w2)
    want = torch.zeros(m, H)
    for i in range(m):
        for k in range(topk):
            e = int(idx[i, k])
            h = x[i].float() @ w13[e].float().t()
            a = (torch.nn.functional.silu(h[:inter]) * h[inter:]).bfloat16().float()
            want[i] += wts[i, k] * (a @ w2[e].float().t()).bfloat16().float()
    torch.testing.assert_close(out.float(), want, rtol=3e-2, atol=3e-2)
