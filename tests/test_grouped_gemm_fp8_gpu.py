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


def _operands(E, rows, K, w_rows, seed, pow2=False):
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(E, rows, K, generator=g)
    w = torch.randn(E, w_rows, K, generator=g) * K ** -0.5
    # Rows with very different magnitudes, so that the scales differ from row to row and from
    # K block to K block (a wrong scale byte then shows as a factor of two or more).
    x = x * torch.exp2(torch.randint(-6, 7, (E, rows, 1), generator=g).float())
    kblocks = (K + 127) // 128
    x = x * torch.exp2(torch.randint(-3, 4, (E, rows, kblocks), generator=g).float()
                       ).repeat_interleave(128, dim=2)[:, :, :K]
    xq, sa = per_token_block_quant(x.view(E * rows, K), pow2=pow2)
    wq, sw = quantize_weight_blocks(w, pow2=pow2)
    return (xq.view(E, rows, K).to(dev), sa.view(E, rows, -1).to(dev), wq.to(dev), sw.to(dev))


@pytest.mark.parametrize("E,rows,K,N,counts", [
    (1, 128, 128, 256, [128]),
    (3, 256, 512, 512, [256, 0, 77]),
    (2, 128, 2048, 768, [100, 128]),       # Qwen3 down projection shape
    (4, 384, 384, 272, [384, 1, 129, 200]),  # column tail, 3 K blocks
])
@pytest.mark.parametrize("pow2", [False, True], ids=["fp32 scales", "power-of-two scales"])
def test_plain_bf16_epilogue(E, rows, K, N, counts, pow2):
    xq, sa, wq, sw = _operands(E, rows, K, N, seed=1, pow2=pow2)
    cnt = torch.tensor(counts, dtype=torch.int32, device=xq.device)
    out = torch.full((E, rows, N), float("nan"), dtype=torch.bfloat16, device=xq.device)
    status = torch.zeros(1, dtype=torch.int32, device=xq.device)
    grouped_gemm_fp8(xq, sa, wq, sw, cnt, out=out, status=status, pow2_scales=pow2)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = grouped_gemm_fp8_reference(xq, sa, wq, sw, cnt)
    for e, m in enumerate(counts):
        tol = 2e-2 * want[e, :m].abs().amax(dim=1, keepdim=True).clamp(min=1.0)
        assert ((out[e, :m].float() - want[e, :m]).abs() <= 2e-2 * want[e, :m].abs() + tol).all()
        assert torch.isnan(out[e, m:].float()).all()


@pytest.mark.parametrize("E,rows,K,I,counts", [
    (1, 128, 256, 128, [128]),
    (2, 256, 2048, 768, [256, 130]),       # Qwen3 up projection shape
    (5, 128, 512, 256, [5, 128, 0, 64, 127]),
])
@pytest.mark.parametrize("pow2", [False, True], ids=["fp32 scales", "power-of-two scales"])
def test_swiglu_epilogue_quantises_its_result(E, rows, K, I, counts, pow2):
    xq, sa, wq, sw = _operands(E, rows, K, 2 * I, seed=2, pow2=pow2)
    cnt = torch.tensor(counts, dtype=torch.int32, device=xq.device)
    status = torch.zeros(1, dtype=torch.int32, device=xq.device)
    hq, hs = grouped_gemm_fp8(xq, sa, wq, sw, cnt, swiglu_quant=True, status=status,
                              pow2_scales=pow2)
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
        if pow2:
            # powers of two, at or just above amax / 448 (the kernel's maximum is of its own
            # fp32 result, which may sit on the other side of a power of two)
            got_s = hs[e, :m].cpu()
            assert torch.equal(got_s, torch.exp2(torch.round(torch.log2(got_s))))
            assert ((got_s >= amax * 0.98) & (got_s <= amax * 2.05)).all()
        else:
            torch.testing.assert_close(hs[e, :m].cpu(), amax, rtol=2e-2, atol=1e-6)


def test_hardware_scaling_reports_a_scale_that_is_not_a_power_of_two():
    """`pow2_scales=True` is a promise; the kernel checks it while it reads the scales and
    reports status 2 instead of silently dropping mantissa bits."""
    xq, sa, wq, sw = _operands(1, 128, 256, 256, seed=5, pow2=False)   # amax / 448: not powers of two
    cnt = torch.tensor([128], dtype=torch.int32, device=xq.device)
    status = torch.zeros(1, dtype=torch.int32, device=xq.device)
    grouped_gemm_fp8(xq, sa, wq, sw, cnt, status=status, pow2_scales=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 2
    status.zero_()
    xq, sa, wq, sw = _operands(1, 128, 256, 256, seed=5, pow2=True)
    grouped_gemm_fp8(xq, sa, wq, sw, cnt, status=status, pow2_scales=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
