"""Numerics of the tcgen05 grouped GEMM against a plain PyTorch fp32 reference."""

import pytest
import torch

from pplx_kernels_b200.ops.grouped_gemm import grouped_gemm, grouped_gemm_reference

pytestmark = pytest.mark.gpu


def _case(E, rows, K, N, counts, swiglu, seed=0, half_n=0, cta_pair=-1):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = (torch.randn(E, rows, K, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    w_rows = 2 * N if swiglu else N
    w = (torch.randn(E, w_rows, K, generator=g) * (K ** -0.5)).to(torch.bfloat16).to(dev)
    cnt = torch.tensor(counts, dtype=torch.int32, device=dev)
    out = torch.full((E, rows, N), float("nan"), dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    grouped_gemm(x, w, cnt, out=out, swiglu=swiglu, status=status, half_n=half_n,
                 cta_pair=cta_pair)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a pipeline wait ran out"
    want = grouped_gemm_reference(x, w, cnt, swiglu)
    for e, m in enumerate(counts):
        torch.testing.assert_close(out[e, :m].float(), want[e, :m], rtol=2e-2, atol=2e-2)
        # rows beyond the count are not written
        assert torch.isnan(out[e, m:].float()).all()


@pytest.mark.parametrize("swiglu", [False, True])
def test_one_expert_one_tile(swiglu):
    _case(E=1, rows=128, K=64, N=256, counts=[128], swiglu=swiglu)


@pytest.mark.parametrize("swiglu", [False, True])
def test_ragged_counts_many_tiles(swiglu):
    _case(E=4, rows=384, K=512, N=512, counts=[384, 0, 130, 1], swiglu=swiglu, seed=1)


def test_k_and_n_tails():
    # K not a multiple of 64 (TMA zero-fills the tail), N not a multiple of 256.
    _case(E=2, rows=256, K=200, N=328, counts=[256, 77], swiglu=False, seed=2)


def test_long_k_wraps_the_stage_ring_many_times():
    _case(E=2, rows=128, K=4096, N=256, counts=[100, 128], swiglu=True, seed=3)


def test_more_tiles_than_sms():
    _case(E=8, rows=512, K=256, N=1536, counts=[512, 500, 3, 512, 256, 129, 0, 512], swiglu=False,
          seed=4)


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("half_n", [64, 72, 112, 120])
def test_narrow_tiles(swiglu, half_n):
    # Tile widths other than 256 columns, with column tails on the last block.
    _case(E=3, rows=256, K=320, N=448, counts=[200, 256, 17], swiglu=swiglu, seed=5, half_n=half_n)


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("cta_pair", [0, 1])
def test_cta_pair_and_single_forms_agree_with_the_reference(swiglu, cta_pair):
    # Row counts around the 128 / 256 tile edges, an empty expert, several K blocks.
    _case(E=5, rows=640, K=448, N=512, counts=[640, 129, 0, 256, 300], swiglu=swiglu, seed=6,
          cta_pair=cta_pair)


def test_cta_pair_long_k_and_narrow_tiles():
    _case(E=2, rows=512, K=2048, N=448, counts=[512, 257], swiglu=True, seed=7, half_n=112,
          cta_pair=1)
