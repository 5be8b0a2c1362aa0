"""Multi-process GPU tests: one process per GPU, peers mapped through CUDA IPC.

Mirrors the reference's `test_all_to_all_4_gpu` (tests/test_all_to_all.py:313-332)
and `test_nvshmem_4_gpu` / `test_all_to_all` of tests/test_nvshmem.py:36-71, at
whatever GPU count the box offers (2, 4 or 8); each test skips when there are
fewer GPUs than it needs.  NVLS is switched off for NCCL in the launcher and the
kernels use plain peer loads/stores.
"""

import pytest
import torch

import pplx_kernels_b200 as pk
from pplx_kernels_b200.utils.testing import MoEConfig, ProcessGroupInfo, parallel_launch

from pplx_kernels_b200.utils.verify import RankBuffers, verify_combine, verify_dispatch, world_inputs

pytestmark = pytest.mark.gpu


def _need(n: int) -> None:
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _init_runtime(pgi: ProcessGroupInfo) -> None:
    from pplx_kernels_b200.parallel.runtime import init_runtime_from_torch

    assert init_runtime_from_torch() == (pgi.rank, pgi.world_size)


def _make(pgi: ProcessGroupInfo, cfg: MoEConfig, dp_size: int, internode: bool) -> pk.AllToAll:
    ctor = pk.AllToAll.internode if internode else pk.AllToAll.intranode
    ata = ctor(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token, pgi.rank,
               pgi.world_size, dp_size, cfg.hidden_dim, cfg.hidden_dim_bytes,
               cfg.hidden_dim_scale_bytes)
    ata.set_debug_checks(True)
    ata.set_timeout_ms(5000)
    return ata


def _worker_all_to_all(pgi: ProcessGroupInfo, cfg: MoEConfig, dp_size: int, internode: bool,
                       iterations: int, split: bool, use_compile: bool = False) -> None:
    if internode:
        _init_runtime(pgi)
    ata = _make(pgi, cfg, dp_size, internode)
    # As in the reference's test (tests/test_all_to_all.py:178, 262): the calls go through
    # torch.compile, which works because the operators have schemas and Meta kernels.
    dispatch = torch.compile(ata.dispatch) if use_compile else ata.dispatch
    combine = torch.compile(ata.combine) if use_compile else ata.combine
    for it in range(iterations):
        inputs = world_inputs(cfg, pgi.world_size, dp_size, seed=100 + it)
        buf = RankBuffers(cfg, pgi.world_size, dp_size, inputs[pgi.rank], pgi.device)
        d = (buf.counts, buf.expert_x, buf.expert_scale, buf.x, buf.x_scale, buf.indices,
             buf.bound_m)
        if split:
            dispatch(*d, do_send=True, do_recv=False)
            dispatch(*d, do_send=False, do_recv=True)
        else:
            dispatch(*d)
        torch.cuda.synchronize()
        ata.check_status()
        verify_dispatch(cfg, inputs, dp_size, pgi.rank, buf)
        buf.make_expert_y()
        c = (buf.out, buf.indices, buf.weights, buf.expert_y, buf.bound_m)
        if split:
            combine(*c, do_send=True, do_recv=False)
            combine(*c, do_send=False, do_recv=True)
        else:
            combine(*c)
        torch.cuda.synchronize()
        ata.check_status()
        verify_combine(cfg, inputs, pgi.rank, buf)
    torch.distributed.barrier()
    ata.destroy()
    if internode:
        pk.nvshmem_finalize()


@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("internode", [False, True])
def test_all_to_all_2_gpu(in_dtype, internode):
    _need(2)
    cfg = MoEConfig(8, 3, 512, 10, in_dtype=in_dtype)
    parallel_launch(2, _worker_all_to_all, cfg, 1, internode, 4, False)


def test_all_to_all_2_gpu_through_torch_compile():
    _need(2)
    cfg = MoEConfig(8, 3, 512, 10, in_dtype=torch.float8_e4m3fn)
    parallel_launch(2, _worker_all_to_all, cfg, 1, False, 3, False, True)


def test_all_to_all_2_gpu_split_mode():
    _need(2)
    cfg = MoEConfig(8, 3, 512, 10, in_dtype=torch.float8_e4m3fn)
    parallel_launch(2, _worker_all_to_all, cfg, 1, False, 3, True)


def test_all_to_all_2_gpu_replicated_tokens():
    _need(2)
    cfg = MoEConfig(8, 3, 512, 10, in_dtype=torch.float8_e4m3fn, out_dtype=torch.float16)
    parallel_launch(2, _worker_all_to_all, cfg, 2, False, 3, False)


@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float8_e4m3fn, torch.float16])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("internode", [True, False])
@pytest.mark.parametrize("use_compile", [False, True])
def test_all_to_all_4_gpu(in_dtype, out_dtype, internode, use_compile):
    """The reference's own matrix (tests/test_all_to_all.py:313-332): world 4, dp 2, three
    input and two output dtypes, both constructors, with and without torch.compile."""
    _need(4)
    cfg = MoEConfig(8, 3, 512, 10, in_dtype=in_dtype, out_dtype=out_dtype)
    parallel_launch(4, _worker_all_to_all, cfg, 2, internode, 2, False, use_compile)


def test_all_to_all_8_gpu_deepseek_shape():
    _need(8)
    cfg = MoEConfig(256, 8, 7168, 32, in_dtype=torch.float8_e4m3fn)
    parallel_launch(8, _worker_all_to_all, cfg, 1, False, 3, False)


# ------------------------------------------------------------ symmetric memory ----


def test_runtime_single_rank():
    uid = pk.nvshmem_get_unique_id()
    pk.nvshmem_init(uid, 0, 1)
    assert pk.nvshmem_my_pe() == 0
    assert pk.nvshmem_n_pes() == 1
    t = pk.nvshmem_malloc([4, 8], torch.float32, torch.device("cuda", 0))
    assert t.shape == (4, 8) and t.is_cuda and float(t.abs().sum()) == 0.0
    pk.nvshmem_barrier_all()
    pk.nvshmem_barrier_all_on_current_stream()
    src = pk.nvshmem_malloc([1, 64], torch.int32, torch.device("cuda", 0))
    dst = pk.nvshmem_malloc([1, 64], torch.int32, torch.device("cuda", 0))
    src.copy_(torch.arange(64, dtype=torch.int32).view(1, 64))
    pk.nvshmem_alltoall(dst, src)
    torch.cuda.synchronize()
    assert torch.equal(dst.cpu(), src.cpu())
    del t, src, dst
    pk.nvshmem_finalize()


def _worker_runtime(pgi: ProcessGroupInfo) -> None:
    _init_runtime(pgi)
    assert pk.nvshmem_my_pe() == pgi.rank
    assert pk.nvshmem_n_pes() == pgi.world_size
    world = pgi.world_size
    t_in = pk.nvshmem_malloc([world, 8], torch.int32, pgi.device)
    t_out = pk.nvshmem_malloc([world, 8], torch.int32, pgi.device)
    t_in.fill_(pgi.rank)
    pk.nvshmem_barrier_all_on_current_stream()
    pk.nvshmem_alltoall(t_out, t_in)
    pk.nvshmem_barrier_all_on_current_stream()
    torch.cuda.synchronize()
    want = torch.arange(world, dtype=torch.int32).view(world, 1).expand(world, 8)
    assert torch.equal(t_out.cpu(), want)
    pk.nvshmem_barrier_all()
    del t_in, t_out
    pk.nvshmem_finalize()


@pytest.mark.parametrize("world", [2, 4])
def test_runtime_alltoall_multi_gpu(world):
    _need(world)
    parallel_launch(world, _worker_runtime)


# ------------------------------------------- driver-allocated arena, multicast ----


def _worker_vmm(pgi: ProcessGroupInfo, cfg: MoEConfig, want_multicast: bool) -> None:
    ata = _make(pgi, cfg, 1, False)
    lay = ata.layout()
    note = ata.multicast_note()
    ata.destroy()
    assert lay["vmm_arena"] == 1, lay
    if want_multicast and pgi.rank == 0:
        print(f"MULTICAST in use: {lay['multicast']} {note!r}", flush=True)
    if not want_multicast:
        assert lay["multicast"] == 0 and note == ""
    # Plain dispatch / combine over the mapped peers, the stream barrier and the dense
    # all-to-all of the runtime, then the fused layer, whose packed send broadcasts its
    # histogram (one multicast store per word where multicast is in use).
    _worker_all_to_all(pgi, cfg, 1, False, 2, False)
    # Tokens replicated on all ranks: with multicast the combine sends every row once.
    _worker_all_to_all(pgi, cfg, pgi.world_size, False, 2, False)
    _worker_runtime(pgi)
    _worker_moe_layer(pgi, "tiny", 48)


@pytest.mark.parametrize("want_multicast", [False, True])
def test_vmm_arena_2_gpu(want_multicast, monkeypatch):
    """The arena as driver allocations passed between the processes as file descriptors
    (PPLX_B200_VMM=1) and, on top, bound to an NVLink multicast object (PPLX_B200_MULTIMEM=1).
    Every rank stays to the end and unbinds before it exits."""
    _need(2)
    monkeypatch.setenv("PPLX_B200_VMM", "1")
    monkeypatch.setenv("PPLX_B200_MULTIMEM", "1" if want_multicast else "0")
    monkeypatch.setenv("PPLX_B200_MULTIMEM_COMBINE", "1")  # on two ranks it is off by default
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    parallel_launch(2, _worker_vmm, MoEConfig(16, 4, 512, 24, in_dtype=torch.bfloat16),
                    want_multicast)


# ---------------------------------------------------------------- lost peer ----


def _worker_lost_peer(pgi: ProcessGroupInfo, cfg: MoEConfig) -> None:
    ata = _make(pgi, cfg, 1, False)
    inputs = world_inputs(cfg, pgi.world_size, 1, seed=7)
    buf = RankBuffers(cfg, pgi.world_size, 1, inputs[pgi.rank], pgi.device)
    d = (buf.counts, buf.expert_x, buf.expert_scale, buf.x, buf.x_scale, buf.indices, buf.bound_m)
    # Step 1: everybody takes part.
    ata.dispatch(*d)
    buf.make_expert_y()
    ata.combine(buf.out, buf.indices, buf.weights, buf.expert_y, buf.bound_m)
    torch.cuda.synchronize()
    ata.check_status()
    torch.distributed.barrier()
    # Step 2: the last rank stays away (between steps, nothing of it in flight).  The others
    # must come back with an error status instead of hanging.
    if pgi.rank != pgi.world_size - 1:
        ata.set_timeout_ms(200)
        ata.dispatch(*d)
        torch.cuda.synchronize()
        st = ata.status()
        assert st["code"] == 1 and st["peer"] == pgi.world_size - 1, st
        with pytest.raises(RuntimeError, match="wait timed out"):
            ata.check_status()
    torch.distributed.barrier()
    ata.destroy()


def test_lost_peer_is_reported_2_gpu():
    _need(2)
    cfg = MoEConfig(8, 2, 256, 8)
    parallel_launch(2, _worker_lost_peer, cfg)


# ------------------------------------------------------------------ MoE layer ----


def _worker_moe_layer(pgi: ProcessGroupInfo, model: str, tokens: int) -> None:
    from pplx_kernels_b200.models.configs import CONFIGS
    from pplx_kernels_b200.models.moe import MoELayer, moe_reference
    from pplx_kernels_b200.utils.testing import as_index_tensor, routing

    cfg = CONFIGS[model]
    dev = pgi.device
    layer = MoELayer(cfg, max_num_tokens=tokens, rank=pgi.rank, world_size=pgi.world_size,
                     device=dev, init_std=0.05)
    layer.ata.set_timeout_ms(5000)
    gen = torch.Generator().manual_seed(50 + pgi.rank)
    x = torch.randn(tokens, cfg.hidden_dim, generator=gen).to(torch.bfloat16).to(dev)
    idx = routing(tokens, cfg.num_experts, cfg.experts_per_token, gen)
    w = torch.softmax(torch.randn(tokens, cfg.experts_per_token, generator=gen), dim=-1).to(dev)
    # The whole model's weights, for the reference: gather every rank's experts.
    w13_all = [torch.empty_like(layer.w13) for _ in range(pgi.world_size)]
    w2_all = [torch.empty_like(layer.w2) for _ in range(pgi.world_size)]
    torch.distributed.all_gather(w13_all, layer.w13)
    torch.distributed.all_gather(w2_all, layer.w2)
    want = moe_reference(x, idx.to(dev), w, torch.cat(w13_all), torch.cat(w2_all))
    for fused in (True, False, True):
        out = layer(x, as_index_tensor(idx, dev), w, fused=fused)
        torch.cuda.synchronize()
        layer.check_status()
        torch.testing.assert_close(out[:tokens].float(), want, rtol=3e-2, atol=3e-3)
    torch.distributed.barrier()
    layer.destroy()


@pytest.mark.parametrize("world", [2, 8])
def test_moe_layer_fused_and_composed_multi_gpu(world):
    _need(world)
    parallel_launch(world, _worker_moe_layer, "tiny", 48)


def _worker_moe_layer_fp8(pgi: ProcessGroupInfo, tokens: int) -> None:
    from pplx_kernels_b200.models.configs import MoEModelConfig
    from pplx_kernels_b200.models.moe import MoELayerFP8, moe_reference_fp8
    from pplx_kernels_b200.utils.testing import as_index_tensor, routing

    cfg = MoEModelConfig("q-multi", 16, 4, 512, 256)
    dev = pgi.device
    layer = MoELayerFP8(cfg, max_num_tokens=tokens, rank=pgi.rank, world_size=pgi.world_size,
                        device=dev, init_std=0.05)
    layer.ata.set_timeout_ms(5000)
    gen = torch.Generator().manual_seed(60 + pgi.rank)
    x = torch.randn(tokens, cfg.hidden_dim, generator=gen).to(torch.bfloat16).to(dev)
    idx = routing(tokens, cfg.num_experts, cfg.experts_per_token, gen)
    w = torch.softmax(torch.randn(tokens, cfg.experts_per_token, generator=gen), dim=-1).to(dev)
    w13, w2 = layer.dequantized_weights()
    w13_all = [torch.empty_like(w13) for _ in range(pgi.world_size)]
    w2_all = [torch.empty_like(w2) for _ in range(pgi.world_size)]
    torch.distributed.all_gather(w13_all, w13)
    torch.distributed.all_gather(w2_all, w2)
    want = moe_reference_fp8(x, idx.to(dev), w, torch.cat(w13_all), torch.cat(w2_all))
    outs = {}
    for fused in (True, False, True):
        out = layer(x, as_index_tensor(idx, dev), w, fused=fused)
        torch.cuda.synchronize()
        layer.check_status()
        got = out[:tokens].float().clone()
        err = (got - want).abs()
        # two e4m3 roundings of the activations on top of bf16
        assert (err <= 0.06 * want.abs() + 0.04 * want.abs().amax()).all(), (fused, err.max())
        outs.setdefault(fused, got)
    # the fused and the composed path do the same arithmetic
    torch.testing.assert_close(outs[True], outs[False], rtol=2e-2, atol=2e-3)
    torch.distributed.barrier()
    layer.destroy()


@pytest.mark.parametrize("world", [2, 8])
def test_fp8_moe_layer_fused_and_composed_multi_gpu(world):
    _need(world)
    parallel_launch(world, _worker_moe_layer_fp8, 48)
