"""CPU tests of the host side: operator surface, configuration checks and the
socket bootstrap (spawned processes, no GPU)."""

import multiprocessing as mp

import pytest
import torch

import pplx_kernels_b200 as pk
from pplx_kernels_b200.ops import _ops


def test_operator_surface_matches_reference_names():
    names = [
        "all_to_all_intranode_create", "all_to_all_internode_create", "all_to_all_destroy",
        "all_to_all_intranode_dispatch", "all_to_all_intranode_combine",
        "all_to_all_internode_dispatch", "all_to_all_internode_combine",
        "nvshmem_get_unique_id", "nvshmem_unique_id_size", "nvshmem_init", "nvshmem_finalize",
        "nvshmem_my_pe", "nvshmem_n_pes", "nvshmem_malloc", "nvshmem_barrier_all",
        "nvshmem_barrier_all_on_current_stream", "nvshmem_alltoall",
    ]
    for n in names:
        assert hasattr(_ops, n), n


def test_dispatch_schema_marks_outputs_mutable():
    schema = str(_ops.all_to_all_intranode_dispatch.default._schema)
    assert "Tensor($0! -> ) out_expert_num_tokens" in schema
    assert "Tensor($2! -> )? out_expert_x_scale" in schema
    assert "Tensor? bound_m" in schema
    schema = str(_ops.all_to_all_internode_combine.default._schema)
    assert "Tensor($0! -> ) out_tokens" in schema


def test_unique_id_is_128_bytes():
    assert pk.nvshmem_unique_id_size() == 128
    uid = pk.nvshmem_get_unique_id()
    assert uid.dtype == torch.uint8 and uid.device.type == "cpu" and uid.numel() == 128
    assert pk.nvshmem_alloc_empty_unique_id().sum() == 0
    assert not torch.equal(uid, pk.nvshmem_get_unique_id())


@pytest.mark.parametrize(
    "kwargs, message",
    [
        (dict(hidden_dim_bytes=1000), "multiple of 16"),
        (dict(hidden_dim_scale_bytes=6), "multiple of 4"),
        (dict(num_experts=0), "num_experts must be positive"),
        (dict(experts_per_token=0), "experts_per_token"),
        (dict(max_num_tokens=0), "max_num_tokens"),
    ],
)
def test_bad_configuration_is_rejected_before_touching_the_gpu(kwargs, message):
    base = dict(max_num_tokens=8, num_experts=8, experts_per_token=2, rank=0, world_size=1,
                dp_size=1, hidden_dim=512, hidden_dim_bytes=1024, hidden_dim_scale_bytes=0)
    base.update(kwargs)
    with pytest.raises(RuntimeError, match=message):
        pk.AllToAll.intranode(**base)


def test_send_and_recv_both_false_is_an_error_name():
    # The op must exist with both flags in its schema (the failure itself needs a GPU object).
    schema = str(_ops.all_to_all_intranode_combine.default._schema)
    assert "bool do_send, bool do_recv" in schema


def _bootstrap_rank(uid_bytes: bytes, rank: int, world: int, q) -> None:
    import torch as t

    from pplx_kernels_b200.ops import _ops as ops

    uid = t.tensor(list(uid_bytes), dtype=t.uint8)
    q.put((rank, ops.bootstrap_selftest(uid, rank, world, 20000).tolist()))


@pytest.mark.parametrize("world", [2, 3])
def test_socket_bootstrap_gathers_and_exchanges(world):
    uid = pk.nvshmem_get_unique_id()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_bootstrap_rank, args=(bytes(uid.tolist()), r, world, q))
             for r in range(1, world)]
    for p in procs:
        p.start()
    mine = _ops.bootstrap_selftest(uid, 0, world, 20000).tolist()
    results = {0: mine}
    for _ in procs:
        r, out = q.get(timeout=60)
        results[r] = out
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        assert results[r][:world] == [1000 + i for i in range(world)]
        assert results[r][world:] == [src * 100 + r for src in range(world)]


def _fd_exchange_rank(uid_bytes: bytes, rank: int, world: int, q) -> None:
    import torch as t

    from pplx_kernels_b200.ops import _ops as ops

    uid = t.tensor(list(uid_bytes), dtype=t.uint8)
    q.put((rank, ops.fd_exchange_selftest(uid, rank, world, 20000).tolist()))


@pytest.mark.parametrize("world", [2, 4])
def test_file_descriptors_travel_between_the_ranks_of_a_box(world):
    """The VMM arena hands its allocations to the peers as file descriptors over unix
    sockets (SCM_RIGHTS); here the descriptors are anonymous files holding one word each."""
    uid = pk.nvshmem_get_unique_id()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_fd_exchange_rank, args=(bytes(uid.tolist()), r, world, q))
             for r in range(1, world)]
    for p in procs:
        p.start()
    results = {0: _ops.fd_exchange_selftest(uid, 0, world, 20000).tolist()}
    for _ in procs:
        r, out = q.get(timeout=60)
        results[r] = out
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    silent = world - 1 if world >= 3 else -1   # this rank passes no descriptor
    for r in range(world):
        want = [-2 if s == r else (-1 if s == silent else 7000 + s) for s in range(world)]
        assert results[r] == want


def test_socket_bootstrap_reports_a_missing_peer():
    # A world of two in which rank 1 never shows up: rank 0 gives up with an error.
    uid = pk.nvshmem_get_unique_id()
    with pytest.raises(RuntimeError, match="peers connected"):
        _ops.bootstrap_selftest(uid, 0, 2, 300)


def test_socket_bootstrap_reports_an_unreachable_hub():
    uid = pk.nvshmem_get_unique_id().clone()
    uid[20:40] = 65  # a socket name nobody listens on
    with pytest.raises(RuntimeError, match="could not reach rank 0"):
        _ops.bootstrap_selftest(uid, 1, 2, 300)


def test_bench_reference_arm_declines_a_single_rank():
    """`bench.py --impl reference` with one rank prints the `unavailable` line and exits 0
    (the reference asserts more than one rank; nothing touches a GPU before that check)."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"],
                         capture_output=True, text=True, timeout=300, env=env, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unavailable"]


def test_cmake_project_configures(tmp_path):
    """The CMake description of the native build configures for sm_100a without a GPU."""
    import os
    import shutil
    import subprocess

    cmake = shutil.which("cmake")
    if cmake is None or shutil.which("ninja") is None:
        pytest.skip("cmake or ninja is not installed")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run(
        [cmake, "-S", os.path.join(root, "pplx_kernels_b200", "csrc"), "-B", str(tmp_path), "-G",
         "Ninja", "-DWITH_TORCH_BINDINGS=OFF", "-DWITH_TESTS=ON", "-DWITH_BENCHMARKS=ON"],
        capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    ninja = (tmp_path / "build.ninja").read_text()
    assert "arch=compute_100a,code=[sm_100a]" in ninja or "sm_100a" in ninja
    assert "test_all_to_all" in ninja and "bench_all_to_all" in ninja


def test_bench_end_to_end_entry_picks_the_best_supported_mode():
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    res = {"e2e_modes_us_per_step": {"eager": 250.0, "graph": None, "host": 200.0},
           "h2d_bytes": 10, "d2h_bytes": 20, "e2e_note": ""}
    e = bench.e2e_entry(8, 128, res)
    assert e["mode"] == "host" and e["us_per_step"] == 200.0
    assert abs(e["value"] - 8 * 128 / 200e-6) < 1e-3
    assert e["modes_us_per_step"]["graph"] is None
    assert e["h2d_bytes_per_step"] == 10 and e["d2h_bytes_per_step"] == 20


def test_bench_compares_with_the_published_numbers_only_at_their_world_size():
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_module2", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.vs_published(1, 128, 1e6) is None
    assert bench.vs_published(8, 7, 1e6) is None
    pub = 8 * 128 / ((83.6 + 102.3) * 1e-6)
    assert abs(bench.vs_published(8, 128, 2 * pub) - 2.0) < 1e-9


def test_helpers_of_the_package_import_without_the_native_library():
    """The benchmark arm that times the unmodified reference imports the package's data and
    clock helpers; that must not map this repository's shared object."""
    import os
    import subprocess
    import sys

    code = ("import pplx_kernels_b200, pplx_kernels_b200.utils.testing, "
            "pplx_kernels_b200.utils.clocks, pplx_kernels_b200.parallel.affinity\n"
            "from pplx_kernels_b200.ops import is_loaded\n"
            "assert not is_loaded()\n"
            "assert 'libpplx_kernels_b200' not in open('/proc/self/maps').read()\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root,
                         timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]


def test_power_of_two_quantisation_oracles():
    """The scales that the hardware-scaled fp8 GEMM takes: powers of two, never below amax / 448,
    below twice that; values survive the round trip within the e4m3 step."""
    import torch

    from pplx_kernels_b200.ops.grouped_gemm import quantize_weight_blocks
    from pplx_kernels_b200.ops.quant import block_dequant, per_token_block_quant

    g = torch.Generator().manual_seed(3)
    x = torch.randn(7, 300, generator=g) * torch.exp2(torch.randint(-8, 8, (7, 1), generator=g).float())
    q, s = per_token_block_quant(x, pow2=True)
    assert s.shape == (7, 3) and torch.equal(s, torch.exp2(torch.round(torch.log2(s))))
    amax = torch.nn.functional.pad(x, (0, 84)).view(7, 3, 128).abs().amax(dim=2).clamp(min=1e-4)
    assert ((s >= amax / 448.0) & (s < 2 * amax / 448.0 * 1.0001)).all()
    back = block_dequant(q, s)
    assert ((back - x).abs() <= 0.0725 * x.abs() + s.repeat_interleave(128, dim=1)[:, :300] * 2 ** -9
            ).all()
    w = torch.randn(2, 130, 200, generator=g)
    wq, ws = quantize_weight_blocks(w, pow2=True)
    assert ws.shape == (2, 2, 2) and torch.equal(ws, torch.exp2(torch.round(torch.log2(ws))))
    full = ws.repeat_interleave(128, dim=1)[:, :130].repeat_interleave(128, dim=2)[:, :, :200]
    assert ((wq.float() * full - w).abs() <= 0.0725 * w.abs() + full * 2 ** -9).all()
