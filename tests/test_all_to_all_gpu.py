"""GPU tests of dispatch/combine.

Single-GPU coverage of the multi-rank protocol comes from local worlds: all
ranks live on GPU 0 and run inside one cooperative launch per operation, with
the same device code as the one-rank-per-GPU path.  The matrix mirrors the
reference's `test_all_to_all_4_gpu` (tests/test_all_to_all.py:313-332: world 4,
dp 2, 8 experts, top-3, hidden 512, three input dtypes x two output dtypes) and
adds what the reference leaves untested: split send/recv, bound_m absent,
strided scales, repeated iterations on one object, EP 1/2/4/8, skewed routing,
CUDA-graph replay and time-outs.
"""

import pytest
import torch

import pplx_kernels_b200 as pk
from pplx_kernels_b200.ops import _ops
from pplx_kernels_b200.utils.testing import MoEConfig, as_index_tensor

from pplx_kernels_b200.utils.verify import (
    RankBuffers,
    run_local_world,
    verify_combine,
    verify_dispatch,
    world_inputs,
)

pytestmark = pytest.mark.gpu


def small(in_dtype=torch.bfloat16, out_dtype=torch.bfloat16, **kw) -> MoEConfig:
    base = dict(num_experts=8, experts_per_token=3, hidden_dim=512, max_num_tokens=10)
    base.update(kw)
    return MoEConfig(in_dtype=in_dtype, out_dtype=out_dtype, **base)


@pytest.fixture(params=["decode-sized kernel", "general kernel"])
def dispatch_kernel_kind(request, monkeypatch):
    """Small objects run the decode-sized dispatch; the same cases must pass on the general
    kernel, which larger objects use."""
    monkeypatch.setenv("PPLX_B200_TINY_MAX_TOKENS",
                       "0" if request.param == "general kernel" else "64")
    return request.param


@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float8_e4m3fn, torch.float16])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
def test_world4_dp2_dtype_matrix(in_dtype, out_dtype, dispatch_kernel_kind):
    run_local_world(small(in_dtype, out_dtype), world=4, dp_size=2, seed=123)


@pytest.mark.parametrize("world,dp_size", [(1, 1), (2, 1), (2, 2), (4, 1), (4, 4), (8, 1), (8, 2)])
def test_expert_parallel_sizes(world, dp_size, dispatch_kernel_kind):
    cfg = small(torch.float8_e4m3fn, num_experts=16, experts_per_token=4, hidden_dim=256,
                max_num_tokens=12)
    run_local_world(cfg, world=world, dp_size=dp_size, seed=5)


@pytest.mark.parametrize("world,dp_size,num_experts", [(4, 1, 10), (4, 2, 7), (8, 1, 9), (2, 1, 5)])
def test_expert_count_that_does_not_divide_evenly(world, dp_size, num_experts):
    """Blocks of ceil(E / W) experts per rank; the last rank(s) own fewer (or none)."""
    cfg = small(torch.float8_e4m3fn, num_experts=num_experts, experts_per_token=3,
                hidden_dim=256, max_num_tokens=12)
    run_local_world(cfg, world=world, dp_size=dp_size, seed=17, iterations=2)


@pytest.mark.parametrize("use_bound_m", [True, False])
@pytest.mark.parametrize("counts", [[0, 5, 0, 12], [0, 0, 0, 0], [1, 0, 0, 0]])
def test_ranks_without_tokens(counts, use_bound_m, dispatch_kernel_kind):
    """bound_m = 0 on some or all ranks: they still post counts, forward what they receive
    and keep their arrival counters in step."""
    cfg = small(torch.float8_e4m3fn, num_experts=16, experts_per_token=4, hidden_dim=256,
                max_num_tokens=12)
    run_local_world(cfg, world=4, dp_size=1, seed=23, iterations=3, num_tokens=counts,
                    use_bound_m=use_bound_m)


def test_float32_expert_outputs():
    run_local_world(small(), world=2, dp_size=1, seed=3, y_dtype=torch.float32)


def test_float32_payload():
    cfg = small(torch.float32, torch.bfloat16, hidden_dim=64)
    run_local_world(cfg, world=2, dp_size=1, seed=4)


def test_tiny_hidden_dim():
    # The reference's C++ test shape: hidden 16, top-3, 8 experts, <= 10 tokens, dp 2.
    cfg = small(torch.bfloat16, torch.bfloat16, hidden_dim=16)
    run_local_world(cfg, world=4, dp_size=2, seed=0xBEEF)


@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float8_e4m3fn])
def test_split_send_recv(in_dtype, dispatch_kernel_kind):
    run_local_world(small(in_dtype), world=4, dp_size=2, seed=11, split=True, iterations=2)


def test_without_bound_m():
    run_local_world(small(torch.float8_e4m3fn), world=4, dp_size=1, seed=12, use_bound_m=False)


def test_strided_scales(dispatch_kernel_kind):
    run_local_world(small(torch.float8_e4m3fn), world=2, dp_size=1, seed=13, strided_scale=True)


def test_many_iterations_on_one_object(dispatch_kernel_kind):
    # Exercises both parities of the flag sets and the self-reset of all counters.
    run_local_world(small(torch.float8_e4m3fn), world=4, dp_size=2, seed=21, iterations=7)


def test_more_tokens_than_blocks():
    # Several tokens per block and several rows per warp.
    cfg = small(torch.bfloat16, num_experts=32, experts_per_token=4, hidden_dim=128,
                max_num_tokens=300)
    run_local_world(cfg, world=4, dp_size=1, seed=31, num_tokens=300, max_blocks=3)


def test_zipf_skewed_routing():
    cfg = small(torch.float8_e4m3fn, num_experts=64, experts_per_token=8, hidden_dim=256,
                max_num_tokens=64)
    run_local_world(cfg, world=8, dp_size=1, seed=41, num_tokens=64, zipf=1.2)


def test_deepseek_shape_world8_emulated():
    cfg = MoEConfig(num_experts=256, experts_per_token=8, hidden_dim=7168, max_num_tokens=16,
                    in_dtype=torch.float8_e4m3fn)
    run_local_world(cfg, world=8, dp_size=1, seed=51, num_tokens=16)


# ---------------------------------------------------------------- single rank ----


def _single_rank(cfg: MoEConfig, seed: int):
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    inputs = world_inputs(cfg, 1, 1, seed)
    ata = pk.AllToAll.intranode(
        cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token, 0, 1, 1, cfg.hidden_dim,
        cfg.hidden_dim_bytes, cfg.hidden_dim_scale_bytes)
    ata.set_debug_checks(True)
    ata.set_timeout_ms(3000)
    buf = RankBuffers(cfg, 1, 1, inputs[0], device)
    return ata, inputs, buf


def _dispatch(ata, buf, **kw):
    ata.dispatch(buf.counts, buf.expert_x, buf.expert_scale, buf.x, buf.x_scale, buf.indices,
                 buf.bound_m, **kw)


def _combine(ata, buf, **kw):
    ata.combine(buf.out, buf.indices, buf.weights, buf.expert_y, buf.bound_m, **kw)


@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float8_e4m3fn])
def test_single_gpu_world_through_public_api(in_dtype):
    cfg = small(in_dtype)
    ata, inputs, buf = _single_rank(cfg, seed=61)
    _dispatch(ata, buf)
    torch.cuda.synchronize()
    verify_dispatch(cfg, inputs, 1, 0, buf)
    buf.make_expert_y()
    _combine(ata, buf)
    torch.cuda.synchronize()
    ata.check_status()
    verify_combine(cfg, inputs, 0, buf)
    ata.destroy()
    ata.destroy()  # idempotent


def test_single_gpu_split_mode_with_work_in_between():
    cfg = small(torch.float8_e4m3fn)
    ata, inputs, buf = _single_rank(cfg, seed=62)
    _dispatch(ata, buf, do_send=True, do_recv=False)
    filler = torch.randn(512, 512, device="cuda") @ torch.randn(512, 512, device="cuda")
    _dispatch(ata, buf, do_send=False, do_recv=True)
    torch.cuda.synchronize()
    verify_dispatch(cfg, inputs, 1, 0, buf)
    buf.make_expert_y()
    _combine(ata, buf, do_send=True, do_recv=False)
    filler = filler @ filler
    _combine(ata, buf, do_send=False, do_recv=True)
    torch.cuda.synchronize()
    ata.check_status()
    verify_combine(cfg, inputs, 0, buf)
    ata.destroy()


def test_send_and_recv_false_is_rejected():
    cfg = small()
    ata, _, buf = _single_rank(cfg, seed=63)
    with pytest.raises(RuntimeError, match="do_send = do_recv = false"):
        _dispatch(ata, buf, do_send=False, do_recv=False)
    ata.destroy()


def test_argument_checks():
    cfg = small(torch.float8_e4m3fn)
    ata, _, buf = _single_rank(cfg, seed=64)
    with pytest.raises(AssertionError):
        ata.dispatch(buf.counts, buf.expert_x, None, buf.x, buf.x_scale, buf.indices, buf.bound_m)
    with pytest.raises(RuntimeError, match="out_expert_num_tokens"):
        ata.dispatch(buf.counts.to(torch.int64), buf.expert_x, buf.expert_scale, buf.x,
                     buf.x_scale, buf.indices, buf.bound_m)
    with pytest.raises(RuntimeError, match="rows per expert"):
        ata.dispatch(buf.counts, buf.expert_x[:, :2].contiguous(), buf.expert_scale[:, :2].contiguous(),
                     buf.x, buf.x_scale, buf.indices, buf.bound_m)
    ata.destroy()
    with pytest.raises(AssertionError):
        _dispatch(ata, buf)


def test_cuda_graph_replay():
    cfg = small(torch.float8_e4m3fn, num_experts=16, experts_per_token=4, hidden_dim=1024,
                max_num_tokens=32)
    ata, inputs, buf = _single_rank(cfg, seed=65)
    # Warm up outside capture, then capture one dispatch + expert + combine round.
    _dispatch(ata, buf)
    buf.make_expert_y()
    _combine(ata, buf)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            _dispatch(ata, buf)
            buf.expert_y.copy_((buf.expert_x.to(torch.float32) * 1.5).to(cfg.out_dtype))
            _combine(ata, buf)
    for n in (3, 1000):
        buf.out.fill_(float("nan"))
        buf.counts.fill_(-1)
        for _ in range(n):
            graph.replay()
        torch.cuda.synchronize()
        ata.check_status()
        verify_dispatch(cfg, inputs, 1, 0, buf)
        verify_combine(cfg, inputs, 0, buf)
    # bound_m is read on the device: shrinking it changes the replayed work.
    new_m = max(1, inputs[0].num_tokens // 2)
    buf.bound_m.view(torch.int32).fill_(new_m)
    inputs[0].num_tokens = new_m
    buf.out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    verify_dispatch(cfg, inputs, 1, 0, buf)
    verify_combine(cfg, inputs, 0, buf)
    ata.destroy()


def test_torch_compile_wraps_the_ops():
    cfg = small(torch.bfloat16)
    ata, inputs, buf = _single_rank(cfg, seed=66)
    dispatch = torch.compile(ata.dispatch)
    combine = torch.compile(ata.combine)
    dispatch(buf.counts, buf.expert_x, buf.expert_scale, buf.x, buf.x_scale, buf.indices,
             buf.bound_m)
    torch.cuda.synchronize()
    verify_dispatch(cfg, inputs, 1, 0, buf)
    buf.make_expert_y()
    combine(buf.out, buf.indices, buf.weights, buf.expert_y, buf.bound_m)
    torch.cuda.synchronize()
    verify_combine(cfg, inputs, 0, buf)
    ata.destroy()


# -------------------------------------------------------------------- time-outs ----


def test_wait_helper_gives_up_and_reports():
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    code, phase, peer, expected, observed = _ops.wait_probe(flag, 20.0)
    assert (code, phase, expected, observed) == (1, 5, 1, 0)
    flag.fill_(7)
    code, *_ = _ops.wait_probe(flag, 20.0)
    assert code == 0
    # the context is still usable
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def test_missing_peer_times_out_instead_of_hanging():
    cfg = small(torch.bfloat16, hidden_dim=64)
    device = torch.device("cuda", 0)
    ranks = pk.AllToAll.local_world(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token,
                                    2, 1, cfg.hidden_dim, cfg.hidden_dim_bytes, 0)
    inputs = world_inputs(cfg, 2, 1, seed=71)
    buf = RankBuffers(cfg, 2, 1, inputs[0], device)
    ranks[0].set_timeout_ms(100)
    # Only rank 0 runs: the counts of rank 1 never arrive.
    pk.dispatch_group([ranks[0]], [buf.counts], [buf.expert_x], [None], [buf.x], [None],
                      [buf.indices], [buf.bound_m])
    torch.cuda.synchronize()
    st = ranks[0].status()
    assert st["code"] == 1 and st["phase"] == 1 and st["peer"] == 1 and st["rank"] == 0
    with pytest.raises(RuntimeError, match="wait timed out"):
        ranks[0].check_status()
    for r in ranks:
        r.destroy()
    # A fresh object works after the failure.
    run_local_world(cfg, world=2, dp_size=1, seed=72)


def test_bad_expert_index_is_reported_with_debug_checks():
    cfg = small(torch.bfloat16, hidden_dim=64)
    ata, inputs, buf = _single_rank(cfg, seed=73)
    bad = buf.indices.view(torch.int32).clone()
    bad[0, 0] = cfg.num_experts + 5
    ata.dispatch(buf.counts, buf.expert_x, None, buf.x, None, bad.view(torch.uint32), buf.bound_m)
    torch.cuda.synchronize()
    st = ata.status()
    assert st["code"] == 2 and st["observed"] == cfg.num_experts + 5
    ata.destroy()


def test_sleep_on_stream_takes_about_that_long():
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _ops.sleep_on_stream(0.002)
    end.record()
    torch.cuda.synchronize()
    assert 1.5 <= start.elapsed_time(end) <= 50.0


# ------------------------------------------------------------ quantising send ----


@pytest.mark.parametrize("world,hidden", [(1, 7168), (4, 1024), (2, 640)])
def test_dispatch_with_fused_fp8_quantisation(world, hidden):
    from pplx_kernels_b200.ops.quant import block_dequant, per_token_block_quant

    from pplx_kernels_b200.ops.reference import simulate_dispatch

    device = torch.device("cuda", 0)
    cfg = MoEConfig(num_experts=16, experts_per_token=4, hidden_dim=hidden, max_num_tokens=24,
                    in_dtype=torch.float8_e4m3fn)
    ranks = pk.AllToAll.local_world(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token,
                                    world, 1, hidden, cfg.hidden_dim_bytes,
                                    cfg.hidden_dim_scale_bytes)
    for r in ranks:
        r.set_debug_checks(True)
        r.set_timeout_ms(3000)
    inputs = world_inputs(cfg, world, 1, seed=81)
    gen = torch.Generator().manual_seed(82)
    xs = [(torch.randn(i.num_tokens, hidden, generator=gen) * 3).to(torch.bfloat16) for i in inputs]
    nle = cfg.num_experts // world
    rows = cfg.max_num_tokens * world
    counts = [torch.full((nle,), -1, dtype=torch.int32, device=device) for _ in range(world)]
    ex = [torch.zeros(nle, rows, hidden, dtype=torch.uint8, device=device).view(torch.float8_e4m3fn)
          for _ in range(world)]
    es = [torch.zeros(nle, rows, cfg.hidden_dim_scale, device=device) for _ in range(world)]
    idx = [as_index_tensor(i.indices, device) for i in inputs]
    if world == 1:
        ranks[0].dispatch_quant(counts[0], ex[0], es[0], xs[0].to(device), idx[0], None)
    else:
        # group launch through the generic op: quantising variant of every rank
        from pplx_kernels_b200.ops import _ops
        _ops.all_to_all_dispatch_quant_group(
            [r._ptr for r in ranks], counts, ex, es, [x.to(device) for x in xs], idx,
            [torch.empty(0, device=device)] * world)
    torch.cuda.synchronize()
    for r in ranks:
        r.check_status()
    expected = simulate_dispatch(inputs, cfg.num_experts, 1)
    for r in range(world):
        assert counts[r].cpu().tolist() == expected[r].counts()
        for le, src_rows in enumerate(expected[r].rows):
            n = len(src_rows)
            if n == 0:
                continue
            want_q, want_s = per_token_block_quant(torch.stack([xs[s][i] for s, i, _ in src_rows]))
            got_q, got_s = ex[r][le, :n].cpu(), es[r][le, :n].cpu()
            # Pair the rows through their scale vectors, which must agree exactly.  A small
            # share of payload bytes may differ by one e4m3 step: bf16 / bf16 ratios land on
            # rounding midpoints surprisingly often, and the host-side float -> e4m3
            # conversion of the oracle does not break those ties the way cvt.rn does.
            order_w = torch.argsort(want_s[:, 0] * 1e3 + want_s[:, -1], stable=True)
            order_g = torch.argsort(got_s[:, 0] * 1e3 + got_s[:, -1], stable=True)
            torch.testing.assert_close(got_s[order_g], want_s[order_w], rtol=1e-6, atol=0)
            gq, wq = got_q[order_g], want_q[order_w]
            mismatch = (gq.view(torch.uint8) != wq.view(torch.uint8)).float().mean().item()
            assert mismatch < 1e-2, f"rank {r} expert {le}: {mismatch:.4f} of the bytes differ"
            torch.testing.assert_close(block_dequant(gq, got_s[order_g]),
                                       block_dequant(wq, want_s[order_w]), rtol=0.13, atol=1e-6)
    # the oracle itself is a faithful quantiser: dequantised values are close to the originals
    q, sc = per_token_block_quant(xs[0])
    rel = (block_dequant(q, sc) - xs[0].float()).abs().max() / xs[0].float().abs().max()
    assert rel < 0.07
    for r in ranks:
        r.destroy()


def test_combine_writes_into_pinned_host_memory():
    """out_tokens in pinned host memory: the reduction stores across PCIe itself and the result
    equals the one written to device memory."""
    cfg = small(torch.bfloat16, num_experts=16, experts_per_token=4, hidden_dim=1024,
                max_num_tokens=32)
    ata, inputs, buf = _single_rank(cfg, seed=71)
    _dispatch(ata, buf)
    buf.make_expert_y()
    _combine(ata, buf)
    torch.cuda.synchronize()
    verify_combine(cfg, inputs, 0, buf)
    want = buf.out.cpu()

    _dispatch(ata, buf)
    host = torch.full(tuple(buf.out.shape), float("nan"), dtype=buf.out.dtype).pin_memory()
    ata.combine(host, buf.indices, buf.weights, buf.expert_y, buf.bound_m)
    torch.cuda.synchronize()
    ata.check_status()
    m = inputs[0].num_tokens
    assert torch.equal(host[:m], want[:m])
    # pageable host memory is refused
    _dispatch(ata, buf)
    with pytest.raises(RuntimeError, match="pinned host"):
        ata.combine(torch.empty(tuple(buf.out.shape), dtype=buf.out.dtype), buf.indices,
                    buf.weights, buf.expert_y, buf.bound_m)
    _combine(ata, buf)
    torch.cuda.synchronize()
    ata.destroy()


def test_dispatch_reads_its_inputs_from_pinned_host_memory():
    """dp_x, dp_x_scale and indices in pinned host memory: the send reads them across PCIe
    itself; counts and rows equal those of the device-input path, and combine takes its weights
    from pinned memory too."""
    cfg = small(torch.float8_e4m3fn, num_experts=16, experts_per_token=4, hidden_dim=1024,
                max_num_tokens=32)
    ata, inputs, buf = _single_rank(cfg, seed=74)
    h_x = buf.x.cpu().pin_memory()
    h_scale = buf.x_scale.cpu().pin_memory()
    h_idx = buf.indices.cpu().pin_memory()
    h_w = buf.weights.cpu().pin_memory()
    for idx in (h_idx, buf.indices):  # the routing table may stay on the device
        buf.counts.fill_(-1)
        buf.expert_x.view(torch.uint8).zero_()
        ata.dispatch(buf.counts, buf.expert_x, buf.expert_scale, h_x, h_scale, idx, buf.bound_m)
        torch.cuda.synchronize()
        ata.check_status()
        verify_dispatch(cfg, inputs, 1, 0, buf)
        buf.make_expert_y()
        buf.out.fill_(float("nan"))
        ata.combine(buf.out, h_idx, h_w, buf.expert_y, buf.bound_m)
        torch.cuda.synchronize()
        ata.check_status()
        verify_combine(cfg, inputs, 0, buf)
    # memory kinds must not be mixed, and pageable memory is refused
    with pytest.raises(RuntimeError, match="same kind of memory"):
        ata.dispatch(buf.counts, buf.expert_x, buf.expert_scale, h_x, buf.x_scale, h_idx,
                     buf.bound_m)
    with pytest.raises(RuntimeError, match="pinned host"):
        ata.dispatch(buf.counts, buf.expert_x, buf.expert_scale, buf.x.cpu(), h_scale, h_idx,
                     buf.bound_m)
    ata.destroy()


def test_host_inputs_with_more_tokens_than_fit_one_staging_round():
    """Blocks that own many tokens fetch them from host memory in several rounds."""
    cfg = MoEConfig(num_experts=8, experts_per_token=2, hidden_dim=4096, max_num_tokens=300,
                    in_dtype=torch.float8_e4m3fn)
    ata, inputs, buf = _single_rank(cfg, seed=75)
    ata.set_max_blocks(3)
    h_x = buf.x.cpu().pin_memory()
    h_scale = buf.x_scale.cpu().pin_memory()
    ata.dispatch(buf.counts, buf.expert_x, buf.expert_scale, h_x, h_scale, buf.indices, buf.bound_m)
    torch.cuda.synchronize()
    ata.check_status()
    verify_dispatch(cfg, inputs, 1, 0, buf)
    buf.make_expert_y()
    _combine(ata, buf)
    torch.cuda.synchronize()
    verify_combine(cfg, inputs, 0, buf)
    ata.destroy()


# ----------------------------------------------------------- both wire protocols ----


def test_flag_in_data_lines_are_the_default_and_can_be_switched_off(monkeypatch):
    cfg = small()
    args = (cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token, 0, 1, 1, cfg.hidden_dim,
            cfg.hidden_dim_bytes, cfg.hidden_dim_scale_bytes)
    monkeypatch.setenv("PPLX_B200_TINY_MAX_TOKENS", str(cfg.max_num_tokens))
    ata = pk.AllToAll.intranode(*args)
    assert ata.layout()["flag_in_data"] == 1 and ata.layout()["decode_sized_dispatch"] == 1
    ata.destroy()
    monkeypatch.setenv("PPLX_B200_TINY_MAX_TOKENS", str(cfg.max_num_tokens - 1))
    ata = pk.AllToAll.intranode(*args)
    assert ata.layout()["flag_in_data"] == 1 and ata.layout()["decode_sized_dispatch"] == 0
    ata.destroy()
    monkeypatch.setenv("PPLX_B200_LL", "0")
    ata = pk.AllToAll.intranode(*args)
    assert ata.layout()["flag_in_data"] == 0
    ata.destroy()
    monkeypatch.delenv("PPLX_B200_LL")
    monkeypatch.setenv("PPLX_B200_LL_MAX_TOKENS", str(cfg.max_num_tokens - 1))
    ata = pk.AllToAll.intranode(*args)
    assert ata.layout()["flag_in_data"] == 0
    ata.destroy()


@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("split", [False, True])
def test_counter_protocol(monkeypatch, in_dtype, split):
    """The store / fence / counter protocol (the one the fused MoE path and the quantising
    send always use) serves the plain calls when the flag-in-data lines are switched off."""
    monkeypatch.setenv("PPLX_B200_LL", "0")
    run_local_world(small(in_dtype), world=4, dp_size=2, seed=81, iterations=3, split=split)
    run_local_world(small(in_dtype), world=8, dp_size=1, seed=82, iterations=2, split=split)


def test_counter_protocol_deepseek_rows(monkeypatch):
    monkeypatch.setenv("PPLX_B200_LL", "0")
    cfg = MoEConfig(num_experts=256, experts_per_token=8, hidden_dim=7168, max_num_tokens=16,
                    in_dtype=torch.float8_e4m3fn)
    run_local_world(cfg, world=8, dp_size=1, seed=83, num_tokens=16)


@pytest.mark.parametrize("hidden", [16, 120, 136, 1016, 2048, 4096])
@pytest.mark.parametrize("in_dtype", [torch.float8_e4m3fn, torch.float32])
def test_row_lengths_around_the_line_size(hidden, in_dtype):
    """Rows that end inside a line, on a line boundary and one chunk past it (a line carries
    120 payload bytes), with the scales spilling into a second meta line at the largest."""
    if in_dtype == torch.float8_e4m3fn and hidden % 16:
        pytest.skip("hidden_dim_bytes must be a multiple of 16")
    cfg = small(in_dtype, hidden_dim=hidden, num_experts=8, experts_per_token=2, max_num_tokens=9)
    run_local_world(cfg, world=2, dp_size=1, seed=84, iterations=2)
    run_local_world(cfg, world=4, dp_size=2, seed=85, split=True, y_dtype=torch.float32)


def test_many_tokens_per_rank_through_lines(monkeypatch):
    monkeypatch.setenv("PPLX_B200_LL_MAX_TOKENS", "0")  # lines at any size
    cfg = MoEConfig(num_experts=32, experts_per_token=4, hidden_dim=2048, max_num_tokens=600,
                    in_dtype=torch.float8_e4m3fn)
    run_local_world(cfg, world=4, dp_size=1, seed=86, iterations=2)


# ------------------------------------------------------- misuse and dead objects ----


def test_two_dispatches_in_a_row_are_refused_on_the_host():
    cfg = small()
    ata, inputs, buf = _single_rank(cfg, seed=87)
    _dispatch(ata, buf)
    with pytest.raises(RuntimeError, match="must alternate"):
        _dispatch(ata, buf)
    buf.make_expert_y()
    with pytest.raises(RuntimeError, match="must alternate"):
        _combine(ata, buf, do_send=False, do_recv=True)
    _combine(ata, buf)
    with pytest.raises(RuntimeError, match="must alternate"):
        _combine(ata, buf)
    torch.cuda.synchronize()
    ata.check_status()
    verify_dispatch(cfg, inputs, 1, 0, buf)
    verify_combine(cfg, inputs, 0, buf)
    ata.destroy()


def test_an_object_refuses_work_after_a_failure_until_it_is_reset():
    """A timed-out wait leaves flags and counters in an unknown state: later calls raise
    instead of returning incomplete data.  The host sees the failure in the pinned mirror of
    the status block without synchronising; reset() on every rank revives the object."""
    cfg = small(torch.bfloat16, hidden_dim=64)
    device = torch.device("cuda", 0)
    ranks = pk.AllToAll.local_world(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token,
                                    2, 1, cfg.hidden_dim, cfg.hidden_dim_bytes, 0)
    inputs = world_inputs(cfg, 2, 1, seed=88)
    bufs = [RankBuffers(cfg, 2, 1, inputs[r], device) for r in range(2)]
    ranks[0].set_timeout_ms(100)

    def dispatch(who):
        pk.dispatch_group([ranks[r] for r in who], [bufs[r].counts for r in who],
                          [bufs[r].expert_x for r in who], [None for _ in who],
                          [bufs[r].x for r in who], [None for _ in who],
                          [bufs[r].indices for r in who], [bufs[r].bound_m for r in who])

    assert ranks[0].peek_status()["code"] == 0
    dispatch([0])  # rank 1 never joins: rank 0's wait for its counts runs out
    torch.cuda.synchronize()
    peek = ranks[0].peek_status()
    assert peek["code"] == 1 and peek["phase"] == 1 and peek["peer"] == 1
    with pytest.raises(RuntimeError, match="recorded a failure earlier"):
        dispatch([0])
    with pytest.raises(RuntimeError, match="recorded a failure earlier"):
        pk.combine_group([ranks[0]], [bufs[0].out], [bufs[0].indices], [bufs[0].weights],
                         [bufs[0].make_expert_y()], [bufs[0].bound_m])
    for r in ranks:
        r.reset()
        r.set_timeout_ms(3000)
        r.set_debug_checks(True)
    assert ranks[0].peek_status()["code"] == 0
    for it in range(2):
        dispatch([0, 1])
        torch.cuda.synchronize()
        for r in range(2):
            ranks[r].check_status()
            verify_dispatch(cfg, inputs, 1, r, bufs[r])
        pk.combine_group(ranks, [b.out for b in bufs], [b.indices for b in bufs],
                         [b.weights for b in bufs], [b.make_expert_y() for b in bufs],
                         [b.bound_m for b in bufs])
        torch.cuda.synchronize()
        for r in range(2):
            ranks[r].check_status()
            verify_combine(cfg, inputs, r, bufs[r])
    for r in ranks:
        r.destroy()


def test_duplicate_experts_in_a_token_are_reported_not_written_past_the_region():
    """The staging region of a source is sized for distinct experts per token.  A token that
    names one expert top-k times on a rank that owns fewer experts than top-k overflows it; the
    send drops the surplus rows and records the overflow whether or not debug checks are on."""
    cfg = small(torch.bfloat16, num_experts=4, experts_per_token=3, hidden_dim=64,
                max_num_tokens=4)
    device = torch.device("cuda", 0)
    ranks = pk.AllToAll.local_world(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token,
                                    2, 1, cfg.hidden_dim, cfg.hidden_dim_bytes, 0)
    inputs = world_inputs(cfg, 2, 1, seed=89, num_tokens=4)
    bufs = [RankBuffers(cfg, 2, 1, inputs[r], device) for r in range(2)]
    bad = torch.zeros(4, 3, dtype=torch.int32, device=device)  # every entry names expert 0
    bufs[0].indices = bad.view(torch.uint32)
    for r in ranks:
        r.set_timeout_ms(300)
    pk.dispatch_group(ranks, [b.counts for b in bufs], [b.expert_x for b in bufs], [None, None],
                      [b.x for b in bufs], [None, None], [b.indices for b in bufs],
                      [b.bound_m for b in bufs])
    torch.cuda.synchronize()
    st = ranks[0].status()
    # kSlotOverflow from the sender, or kRowOverflow from a receiving block that saw the
    # oversized count first
    assert st["code"] in (3, 4), st
    ranks[0].verify_canaries()
    ranks[1].verify_canaries()
    for r in ranks:
        r.destroy()


def test_world_graph_replayed_with_a_changing_bound_m(dispatch_kernel_kind):
    """All ranks of an emulated world inside one CUDA graph (dispatch, expert, combine),
    replayed many times; bound_m of one DP group changes between replays.  Graph replay across
    ranks is what leans hardest on the iteration-numbered flags."""
    cfg = small(torch.float8_e4m3fn, num_experts=16, experts_per_token=4, hidden_dim=1024,
                max_num_tokens=24)
    world, dp_size = 4, 1
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    ranks = pk.AllToAll.local_world(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token,
                                    world, dp_size, cfg.hidden_dim, cfg.hidden_dim_bytes,
                                    cfg.hidden_dim_scale_bytes)
    for r in ranks:
        r.set_timeout_ms(3000)
    inputs = world_inputs(cfg, world, dp_size, seed=90, num_tokens=24)
    bufs = [RankBuffers(cfg, world, dp_size, inputs[r], device) for r in range(world)]
    for b in bufs:
        b.make_expert_y()

    def step():
        pk.dispatch_group(ranks, [b.counts for b in bufs], [b.expert_x for b in bufs],
                          [b.expert_scale for b in bufs], [b.x for b in bufs],
                          [b.x_scale for b in bufs], [b.indices for b in bufs],
                          [b.bound_m for b in bufs])
        for b in bufs:
            b.expert_y.copy_((b.expert_x.to(torch.float32) * 1.5).to(cfg.out_dtype))
        pk.combine_group(ranks, [b.out for b in bufs], [b.indices for b in bufs],
                         [b.weights for b in bufs], [b.expert_y for b in bufs],
                         [b.bound_m for b in bufs])

    step()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            step()
    try:
        for replays, m1 in ((1000, 24), (3, 7), (50, 0), (5, 19)):
            bufs[1].bound_m.view(torch.int32).fill_(m1)
            inputs[1].num_tokens = m1
            for b in bufs:
                b.out.fill_(float("nan"))
                b.counts.fill_(-1)
            for _ in range(replays):
                graph.replay()
            torch.cuda.synchronize()
            for r in range(world):
                ranks[r].check_status()
                verify_dispatch(cfg, inputs, dp_size, r, bufs[r])
                verify_combine(cfg, inputs, r, bufs[r])
    finally:
        for r in ranks:
            r.destroy()


def test_a_rank_may_run_one_dispatch_ahead_of_a_peer(dispatch_kernel_kind):
    """Rank S, whose tokens of step n use none of rank A's experts, finishes its combine
    without waiting for A and sends the rows of dispatch n + 1 to A before A has read the
    rows of dispatch n.  Flags and staging are kept per parity, so A still receives step n
    intact."""
    from pplx_kernels_b200.ops.reference import RankInputs

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    cfg = small(torch.bfloat16, num_experts=8, experts_per_token=2, hidden_dim=256,
                max_num_tokens=6)
    gen = torch.Generator().manual_seed(91)

    def make(m: int, lo: int, hi: int) -> RankInputs:
        idx = torch.stack([lo + torch.randperm(hi - lo, generator=gen)[:2] for _ in range(m)])
        return RankInputs(x=torch.randn(m, cfg.hidden_dim, generator=gen).to(cfg.in_dtype),
                          x_scale=None, indices=idx.to(torch.int64),
                          weights=torch.rand(m, 2, generator=gen), num_tokens=m)

    A, S = 0, 1  # A owns experts 0-3, S owns experts 4-7
    step_n = [make(5, 0, 8), make(6, 4, 8)]      # S's tokens stay on S's own experts
    step_n1 = [make(4, 0, 8), make(6, 0, 4)]     # now every row of S goes to A
    ranks = pk.AllToAll.local_world(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token,
                                    2, 1, cfg.hidden_dim, cfg.hidden_dim_bytes,
                                    cfg.hidden_dim_scale_bytes)
    try:
        for r in ranks:
            r.set_debug_checks(True)
            r.set_timeout_ms(3000)
        bn = [RankBuffers(cfg, 2, 1, step_n[r], device) for r in range(2)]
        bn1 = [RankBuffers(cfg, 2, 1, step_n1[r], device) for r in range(2)]

        def dispatch(who, bufs, **kw):
            pk.dispatch_group([ranks[r] for r in who], [bufs[r].counts for r in who],
                              [bufs[r].expert_x for r in who], [None for _ in who],
                              [bufs[r].x for r in who], [None for _ in who],
                              [bufs[r].indices for r in who], [bufs[r].bound_m for r in who],
                              **kw)

        def combine(who, bufs, **kw):
            pk.combine_group([ranks[r] for r in who], [bufs[r].out for r in who],
                             [bufs[r].indices for r in who], [bufs[r].weights for r in who],
                             [bufs[r].expert_y for r in who], [bufs[r].bound_m for r in who],
                             **kw)

        def check(who):
            torch.cuda.synchronize()
            for r in who:
                ranks[r].check_status()

        dispatch([A, S], bn, do_send=True, do_recv=False)
        dispatch([S], bn, do_send=False, do_recv=True)
        check([S])
        verify_dispatch(cfg, step_n, 1, S, bn[S])
        bn[S].make_expert_y()
        combine([S], bn, do_send=True, do_recv=False)
        combine([S], bn, do_send=False, do_recv=True)
        check([S])
        verify_combine(cfg, step_n, S, bn[S])

        dispatch([S], bn1, do_send=True, do_recv=False)   # S is one dispatch ahead of A
        check([S])

        dispatch([A], bn, do_send=False, do_recv=True)    # A reads step n only now
        check([A])
        verify_dispatch(cfg, step_n, 1, A, bn[A])
        bn[A].make_expert_y()
        combine([A], bn, do_send=True, do_recv=False)
        combine([A], bn, do_send=False, do_recv=True)
        check([A])
        verify_combine(cfg, step_n, A, bn[A])

        dispatch([A], bn1, do_send=True, do_recv=False)
        dispatch([A, S], bn1, do_send=False, do_recv=True)
        check([A, S])
        for r in (A, S):
            verify_dispatch(cfg, step_n1, 1, r, bn1[r])
            bn1[r].make_expert_y()
        combine([A, S], bn1)
        check([A, S])
        for r in (A, S):
            verify_combine(cfg, step_n1, r, bn1[r])
    finally:
        for r in ranks:
            r.destroy()
