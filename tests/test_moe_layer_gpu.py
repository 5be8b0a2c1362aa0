"""The MoE layer (dispatch -> tcgen05 grouped GEMMs -> combine) against plain PyTorch."""

import pytest
import torch

from pplx_kernels_b200.models.configs import TINY, MoEModelConfig
from pplx_kernels_b200.models.moe import MoELayer, moe_reference
from pplx_kernels_b200.utils.testing import as_index_tensor, routing

pytestmark = pytest.mark.gpu


def _inputs(cfg: MoEModelConfig, m: int, seed: int, dev):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(m, cfg.hidden_dim, generator=gen).to(torch.bfloat16)
    idx = routing(m, cfg.num_experts, cfg.experts_per_token, gen)
    w = torch.softmax(torch.randn(m, cfg.experts_per_token, generator=gen), dim=-1)
    return x.to(dev), idx, w.to(dev)


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("cfg,m", [(TINY, 40), (MoEModelConfig("t2", 4, 2, 512, 256), 200),
                                   (MoEModelConfig("t3", 2, 2, 256, 256), 300)])
def test_single_rank_layer_matches_reference(cfg, m, fused):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    layer = MoELayer(cfg, max_num_tokens=m, init_std=0.05)
    x, idx, w = _inputs(cfg, m, seed=3, dev=dev)
    out = layer(x, as_index_tensor(idx, dev), w, fused=fused)
    torch.cuda.synchronize()
    layer.check_status()
    want = moe_reference(x, idx.to(dev), w, layer.w13, layer.w2)
    torch.testing.assert_close(out[:m].float(), want, rtol=3e-2, atol=3e-3)
    # a second pass on the same object (flag parity, counters) gives the same answer
    out2 = layer(x, as_index_tensor(idx, dev), w, fused=not fused)
    torch.cuda.synchronize()
    torch.testing.assert_close(out2[:m].float(), want, rtol=3e-2, atol=3e-3)
    out3 = layer(x, as_index_tensor(idx, dev), w, fused=fused)
    torch.cuda.synchronize()
    torch.testing.assert_close(out3[:m], out[:m])
    layer.destroy()


def test_layer_in_a_cuda_graph():
    cfg, m = TINY, 32
    dev = torch.device("cuda", 0)
    layer = MoELayer(cfg, max_num_tokens=m, init_std=0.05)
    x, idx, w = _inputs(cfg, m, seed=4, dev=dev)
    idx_dev = as_index_tensor(idx, dev)
    out = torch.zeros(m, cfg.hidden_dim, dtype=torch.bfloat16, device=dev)
    layer(x, idx_dev, w, out=out)  # warm-up outside capture
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream), torch.cuda.graph(graph, stream=stream):
        layer(x, idx_dev, w, out=out)
    out.zero_()
    for _ in range(50):
        graph.replay()
    torch.cuda.synchronize()
    layer.check_status()
    want = moe_reference(x, idx.to(dev), w, layer.w13, layer.w2)
    torch.testing.assert_close(out.float(), want, rtol=3e-2, atol=3e-3)
    layer.destroy()


@pytest.mark.parametrize("world,dp_size,m", [(2, 1, 24), (4, 2, 24), (2, 1, 400)])
def test_fused_layer_in_an_emulated_world(world, dp_size, m):
    """All ranks on one GPU.  Every step is launched for all ranks before the next step
    begins, so no kernel ever waits for a later launch."""
    import pplx_kernels_b200 as pk

    # For m = 400 a large row hint selects the CTA-pair form of both GEMMs.
    cfg = TINY
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    expect = (1 << 20) if m >= 400 else m * cfg.experts_per_token // dp_size
    atas = pk.AllToAll.local_world(m, cfg.num_experts, cfg.experts_per_token, world, dp_size,
                                   cfg.hidden_dim, cfg.hidden_dim * 2, 0)
    layers = [MoELayer(cfg, m, rank=r, world_size=world, dp_size=dp_size, device=dev,
                       ata=atas[r], init_std=0.05) for r in range(world)]
    for a in atas:
        a.set_debug_checks(True)
        a.set_timeout_ms(2000)
    groups = world // dp_size
    data = [_inputs(cfg, m, seed=10 + g, dev=dev) for g in range(groups)]
    per_rank = [data[r // dp_size] for r in range(world)]
    idx_dev = [as_index_tensor(d[1], dev) for d in per_rank]
    outs = [torch.full((m, cfg.hidden_dim), float("nan"), dtype=torch.bfloat16, device=dev)
            for _ in range(world)]
    w13 = torch.cat([l.w13 for l in layers])
    w2 = torch.cat([l.w2 for l in layers])
    for _ in range(3):  # several rounds on the same objects
        for o in outs:
            o.fill_(float("nan"))
        pk.fused_dispatch_group(atas, [d[0] for d in per_rank], idx_dev, [None] * world)
        for l in layers:
            l.ata.fused_up(l.w13, l.h, l.counts, l.gemm_status, expect)
        for l in layers:
            l.ata.fused_down(l.h, l.w2, l.gemm_status, expect)
        pk.combine_group(atas, outs, idx_dev, [d[2] for d in per_rank],
                         [l.expert_y for l in layers], [None] * world,
                         do_send=False, do_recv=True)
        torch.cuda.synchronize()
        for r, l in enumerate(layers):
            l.check_status()
            x, idx, w = per_rank[r]
            want = moe_reference(x, idx.to(dev), w, w13, w2)
            torch.testing.assert_close(outs[r].float(), want, rtol=3e-2, atol=3e-3)
    # the per-expert totals reported by the fused up projection
    total = sum(int(l.counts.sum()) for l in layers)
    assert total == groups * m * cfg.experts_per_token
    for l in layers:
        l.destroy()


@pytest.mark.parametrize("pow2", [False, True], ids=["fp32 scales", "power-of-two scales"])
def test_fp8_layer_matches_reference(pow2):
    from pplx_kernels_b200.models.moe import MoELayerFP8, moe_reference_fp8

    cfg, m = MoEModelConfig("q", 8, 2, 512, 256), 96
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    layer = MoELayerFP8(cfg, max_num_tokens=m, init_std=0.05, pow2_scales=pow2)
    x, idx, w = _inputs(cfg, m, seed=21, dev=dev)
    want = moe_reference_fp8(x, idx.to(dev), w, *layer.dequantized_weights(), pow2=pow2)
    for _ in range(2):
        out = layer(x, as_index_tensor(idx, dev), w)
        torch.cuda.synchronize()
        layer.check_status()
        # two e4m3 roundings of the activations on top of bf16: a few percent of the row scale
        err = (out[:m].float() - want).abs()
        assert (err <= 0.06 * want.abs() + 0.03 * want.abs().amax()).all(), err.max()
    layer.destroy()


@pytest.mark.parametrize("cfg,m", [(MoEModelConfig("q", 8, 2, 512, 256), 96),
                                   (MoEModelConfig("q3", 16, 4, 1024, 384), 300)])
@pytest.mark.parametrize("pow2", [False, True], ids=["fp32 scales", "power-of-two scales"])
def test_fused_fp8_layer_matches_reference(cfg, m, pow2):
    """One rank: quantising packed send -> fp8 up projection fed from the staging arena (rows
    and scales) -> fp8 down projection storing into the combine staging -> reduction."""
    from pplx_kernels_b200.models.moe import MoELayerFP8, moe_reference_fp8

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    layer = MoELayerFP8(cfg, max_num_tokens=m, init_std=0.05, pow2_scales=pow2)
    x, idx, w = _inputs(cfg, m, seed=23, dev=dev)
    want = moe_reference_fp8(x, idx.to(dev), w, *layer.dequantized_weights(), pow2=pow2)
    idx_dev = as_index_tensor(idx, dev)
    composed = layer(x, idx_dev, w).clone()
    for _ in range(3):
        out = layer(x, idx_dev, w, fused=True)
        torch.cuda.synchronize()
        layer.check_status()
        err = (out[:m].float() - want).abs()
        assert (err <= 0.06 * want.abs() + 0.03 * want.abs().amax()).all(), err.max()
        # same arithmetic as the composed path: the two must agree to rounding of the sums
        torch.testing.assert_close(out[:m].float(), composed[:m].float(), rtol=2e-2, atol=2e-3)
    assert int(layer.counts.sum()) == m * cfg.experts_per_token
    layer.destroy()


@pytest.mark.parametrize("world,dp_size,m", [(2, 1, 24), (4, 2, 40), (8, 1, 64)])
@pytest.mark.parametrize("pow2", [False, True], ids=["fp32 scales", "power-of-two scales"])
def test_fused_fp8_layer_in_an_emulated_world(world, dp_size, m, pow2):
    """All ranks on one GPU, each step launched for all ranks before the next one."""
    import pplx_kernels_b200 as pk
    from pplx_kernels_b200.models.moe import MoELayerFP8, moe_reference_fp8

    cfg = MoEModelConfig("q4", 16, 4, 512, 256)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    nscale = (cfg.hidden_dim + 127) // 128
    atas = pk.AllToAll.local_world(m, cfg.num_experts, cfg.experts_per_token, world, dp_size,
                                   cfg.hidden_dim, cfg.hidden_dim, nscale * 4)
    layers = [MoELayerFP8(cfg, m, rank=r, world_size=world, dp_size=dp_size, device=dev,
                          ata=atas[r], init_std=0.05, pow2_scales=pow2) for r in range(world)]
    for a in atas:
        a.set_debug_checks(True)
        a.set_timeout_ms(2000)
    groups = world // dp_size
    data = [_inputs(cfg, m, seed=30 + g, dev=dev) for g in range(groups)]
    per_rank = [data[r // dp_size] for r in range(world)]
    idx_dev = [as_index_tensor(d[1], dev) for d in per_rank]
    outs = [torch.full((m, cfg.hidden_dim), float("nan"), dtype=torch.bfloat16, device=dev)
            for _ in range(world)]
    deq = [l.dequantized_weights() for l in layers]
    w13 = torch.cat([d[0] for d in deq])
    w2 = torch.cat([d[1] for d in deq])
    for _ in range(3):
        for o in outs:
            o.fill_(float("nan"))
        pk.fused_dispatch_group(atas, [d[0] for d in per_rank], idx_dev, [None] * world,
                                quantize=True)
        for l in layers:
            l.ata.fused_up_fp8(l.w13_q, l.w13_s, l.h, l.h_scale, l.counts, l.gemm_status)
        for l in layers:
            l.ata.fused_down_fp8(l.h, l.h_scale, l.w2_q, l.w2_s, l.gemm_status)
        pk.combine_group(atas, outs, idx_dev, [d[2] for d in per_rank],
                         [l.expert_y for l in layers], [None] * world,
                         do_send=False, do_recv=True)
        torch.cuda.synchronize()
        for r, l in enumerate(layers):
            l.check_status()
            x, idx, w = per_rank[r]
            want = moe_reference_fp8(x, idx.to(dev), w, w13, w2, pow2=pow2)
            err = (outs[r].float() - want).abs()
            assert (err <= 0.06 * want.abs() + 0.03 * want.abs().amax()).all(), err.max()
    total = sum(int(l.counts.sum()) for l in layers)
    assert total == groups * m * cfg.experts_per_token
    for l in layers:
        l.destroy()


def test_fp8_layer_graph_replayed_1000_times():
    from pplx_kernels_b200.models.moe import MoELayerFP8, moe_reference_fp8

    cfg, m = MoEModelConfig("q2", 16, 4, 256, 128), 16
    dev = torch.device("cuda", 0)
    layer = MoELayerFP8(cfg, max_num_tokens=m, init_std=0.05)
    x, idx, w = _inputs(cfg, m, seed=22, dev=dev)
    idx_dev = as_index_tensor(idx, dev)
    out = torch.zeros(m, cfg.hidden_dim, dtype=torch.bfloat16, device=dev)
    layer(x, idx_dev, w, out=out)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream), torch.cuda.graph(graph, stream=stream):
        layer(x, idx_dev, w, out=out)
    out.zero_()
    for _ in range(1000):
        graph.replay()
    torch.cuda.synchronize()
    layer.check_status()
    want = moe_reference_fp8(x, idx.to(dev), w, *layer.dequantized_weights())
    err = (out.float() - want).abs()
    assert (err <= 0.06 * want.abs() + 0.03 * want.abs().amax()).all(), err.max()
    layer.destroy()
