"""Numerics of the block-scaled fp8 grouped GEMM against a plain PyTorch fp32 reference."""

import pytest
import torch

from pplx_kernels_b200.ops.grouped_gemm import (
    grouped_gemm_fp8,
    grouped_gemm_fp8_reference,
    quantize_weight_blocks,
)
from pplx_kernels_b200.ops.quant import block_dequant, per_token_block_quant

pytestmark = pytest.mark.gpu


def _operands(E, rows, K, w_rows, seed):
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(E, rows, K, generator=g)
    w = torch.randn(E, w_rows, K, generator=g) * K ** -0.5
    xq, sa = per_token_block_quant(x.view(E * rows, K))
    wq, sw = quantize_weight_blocks(w)
    return (xq.view(E, rows, K).to(dev), sa.view(E, rows, -1).to(dev), wq.to(dev), sw.to(dev))


@pytest.mark.parametrize("E,rows,K,N,counts", [
    (1, 128, 128, 256, [128]),
    (3, 256, 512, 512, [256, 0, 77]),
    (2, 128, 2048, 768, [100, 128]),       # Qwen3 down projection shape
    (4, 384, 384, 272, [384, 1, 129, 200]),  # column tail, 3 K blocks
])
def test_plain_bf16_epilogue(E, rows, K, N, counts):
    xq, sa, wq, sw = _operands(E, rows, K, N, seed=1)
    cnt = torch.tensor(counts, dtype=torch.int32, device=xq.device)
    out = torch.full((E, rows, N), float("nan"), dtype=torch.bfloat16, device=xq.device)
    status = torch.zeros(1, dtype=torch.int32, device=xq.device)
    grouped_gemm_fp8(xq, sa, wq, sw, cnt, out=out, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = grouped_gemm_fp8_reference(xq, sa, wq, sw, cnt)
    for e, m in enumerate(counts):
        torch.testing.assert_close(out[e, :m].float(), want[e, :m], rtol=2e-2, atol=2e-2)
        assert torch.isnan(out[e, m:].float()).all()


@pytest.mark.parametrize("E,rows,K,I,counts", [
    (1, 128, 256, 128, [128]),
    (2, 256, 2048, 768, [256, 130]),       # Qwen3 up projection shape
    (5, 128, 512, 256, [5, 128, 0, 64, 127]),
])
def test_swiglu_epilogue_quantises_its_result(E, rows, K, I, counts):
    xq, sa, wq, sw = _operands(E, rows, K, 2 * I, seed=2)
    cnt = torch.tensor(counts, dtype=torch.int32, device=xq.device)
    status = torch.zeros(1, dtype=torch.int32, device=xq.device)
    hq, hs = grouped_gemm_fp8(xq, sa, wq, sw, cnt, swiglu_quant=True, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = grouped_gemm_fp8_reference(xq, sa, wq, sw, cnt, swiglu=True)
    for e, m in enumerate(counts):
        if m == 0:
            continue
        got = block_dequant(hq[e, :m].cpu(), hs[e, :m].cpu())
        w = want[e, :m].cpu()
        # e4m3 keeps 3 mantissa bits: 6.25 % relative step, plus the scale floor
        assert ((got - w).abs() <= 0.07 * w.abs() + 0.02 * w.abs().amax(dim=1, keepdim=True)).all()
        # the scales are the per-block maxima of the result
        amax = w.view(m, -1, 128).abs().amax(dim=2).clamp(min=1e-4) / 448.0
        torch.testing.assert_close(hs[e, :m].cpu(), amax, rtol=2e-2, atol=1e-6)
