"""GPU test of the allocation-free single-rank dispatch entry point.

Some callers of this library cannot allocate device memory: code running under
a stream capture of a framework that forbids allocation while capturing, serving
loops whose device memory is all handed out at start-up, and plugins that only receive
tensors and a stream.  For them the library exports one C function,
``pplx_b200_dispatch_single_rank_noalloc``, whose staging memory is a fixed
16 MiB array inside the library image.  This test calls it through its exported
C symbol (ctypes, raw device pointers) and checks that it produces what the
regular ``AllToAll.dispatch`` produces for a one-rank world: equal per-expert
counts and, per expert, the same rows (payload joined with its scales) as a
multiset -- row order inside an expert is unspecified for both.  It does so
twice in a row with different routing, because every call reuses the same array
and must not be confused by what the previous call left there.

The file name sorts last on purpose, so a run that stops at the first failure
has already run every other test.
"""

import ctypes

import pytest
import torch

import pplx_kernels_b200 as pk
from pplx_kernels_b200.ops import library_path
from pplx_kernels_b200.ops.reference import simulate_dispatch
from pplx_kernels_b200.utils.testing import MoEConfig, as_index_tensor, make_rank_inputs
from pplx_kernels_b200.utils.verify import _joined_rows, _sorted_rows

pytestmark = pytest.mark.gpu

_I64, _INT, _PTR = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p


def _entry_point():
    lib = ctypes.CDLL(str(library_path()))
    fn = lib.pplx_b200_dispatch_single_rank_noalloc
    fn.restype = _INT
    fn.argtypes = [
        _PTR, _PTR, _I64, _I64, _I64,          # counts, out_x, strides, rows per expert
        _PTR, _I64, _I64, _I64,                # out_scale + strides
        _PTR, _I64, _PTR, _I64, _I64,          # x, stride, x_scale + strides
        _PTR, _PTR, _INT, _INT, _INT, _INT, _INT,  # indices, bound_m, m, E, topk, bytes, scale bytes
        _PTR, _PTR, ctypes.c_char_p, ctypes.c_size_t,  # status, stream, message buffer
    ]
    return fn


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _call(fn, cfg, counts, out_x, out_scale, x, x_scale, indices, bound_m, status, num_tokens=None):
    msg = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(
        _ptr(counts), _ptr(out_x), out_x.stride(0) * out_x.element_size(),
        out_x.stride(1) * out_x.element_size(), out_x.size(1),
        _ptr(out_scale), *(out_scale.stride() if out_scale is not None else (0, 0, 0)),
        _ptr(x), x.stride(0) * x.element_size(),
        _ptr(x_scale), *(x_scale.stride() if x_scale is not None else (0, 0)),
        _ptr(indices), _ptr(bound_m), indices.size(0) if num_tokens is None else num_tokens,
        cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim_bytes, cfg.hidden_dim_scale_bytes,
        _ptr(status), ctypes.c_void_p(stream), msg, len(msg))
    return rc, msg.value.decode()


def _outputs(cfg, device):
    counts = torch.full((cfg.num_experts,), -7, dtype=torch.int32, device=device)
    out_x = torch.zeros(cfg.num_experts, cfg.max_num_tokens, cfg.hidden_dim, dtype=torch.uint8,
                        device=device).view(cfg.in_dtype) if cfg.in_dtype.itemsize == 1 else \
        torch.zeros(cfg.num_experts, cfg.max_num_tokens, cfg.hidden_dim, dtype=cfg.in_dtype,
                    device=device)
    out_scale = None
    if cfg.hidden_dim_scale:
        out_scale = torch.zeros(cfg.num_experts, cfg.max_num_tokens, cfg.hidden_dim_scale,
                                device=device)
    return counts, out_x, out_scale


def _assert_same_dispatch(cfg, got, want):
    g_counts, g_x, g_scale = got
    w_counts, w_x, w_scale = want
    assert g_counts.cpu().tolist() == w_counts.cpu().tolist()
    for e, n in enumerate(w_counts.cpu().tolist()):
        if n == 0:
            continue
        g = _sorted_rows(_joined_rows(g_x[e, :n].cpu(), g_scale[e, :n].cpu() if g_scale is not None else None))
        w = _sorted_rows(_joined_rows(w_x[e, :n].cpu(), w_scale[e, :n].cpu() if w_scale is not None else None))
        assert torch.equal(g, w), f"expert {e}: rows differ from the regular dispatch"


@pytest.mark.parametrize("in_dtype", [torch.float8_e4m3fn, torch.bfloat16])
def test_matches_regular_dispatch_on_two_calls_in_a_row(in_dtype):
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    cfg = MoEConfig(num_experts=32, experts_per_token=4, hidden_dim=1024, max_num_tokens=48,
                    in_dtype=in_dtype)
    fn = _entry_point()
    ata = pk.AllToAll.intranode(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token, 0, 1,
                                1, cfg.hidden_dim, cfg.hidden_dim_bytes,
                                cfg.hidden_dim_scale_bytes)
    status = torch.full((1,), 9, dtype=torch.int32, device=device)
    # The first call does the once-per-device set-up; it happens here, outside any capture.
    for call, (seed, tokens) in enumerate([(1, 48), (2, 17)]):
        inp = make_rank_inputs(cfg, torch.Generator().manual_seed(seed), num_tokens=tokens)
        x = inp.x.to(device)
        x_scale = inp.x_scale.to(device) if inp.x_scale is not None else None
        indices = as_index_tensor(inp.indices, device)
        bound_m = torch.tensor([tokens], dtype=torch.int32, device=device)

        want = _outputs(cfg, device)
        ata.dispatch(want[0], want[1], want[2], x, x_scale, indices, bound_m.view(torch.uint32))
        got = _outputs(cfg, device)
        rc, msg = _call(fn, cfg, got[0], got[1], got[2], x, x_scale, indices, bound_m, status)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert int(status.item()) == 0, f"call {call}: the kernel reported a timed-out wait"
        _assert_same_dispatch(cfg, got, want)
        # ... and what the pure-PyTorch oracle says a one-rank dispatch delivers.
        oracle = simulate_dispatch([inp], cfg.num_experts, 1)[0]
        assert got[0].cpu().tolist() == oracle.counts()
        for e, rows in enumerate(oracle.rows):
            if not rows:
                continue
            w_x = torch.stack([inp.x[i] for _, i, _ in rows])
            w_s = torch.stack([inp.x_scale[i] for _, i, _ in rows]) if inp.x_scale is not None else None
            g_s = got[2][e, :len(rows)].cpu() if got[2] is not None else None
            assert torch.equal(_sorted_rows(_joined_rows(got[1][e, :len(rows)].cpu(), g_s)),
                               _sorted_rows(_joined_rows(w_x, w_s))), f"expert {e}: rows differ from the oracle"
        # The regular path must be left in a state from which combine works: finish the round.
        out = torch.empty(cfg.max_num_tokens, cfg.hidden_dim, dtype=torch.bfloat16, device=device)
        ata.combine(out, indices, inp.weights.to(device), want[1].to(torch.bfloat16),
                    bound_m.view(torch.uint32))
        torch.cuda.synchronize()
    ata.check_status()
    ata.destroy()


def test_bound_m_is_optional_and_read_on_the_device():
    device = torch.device("cuda", 0)
    cfg = MoEConfig(num_experts=8, experts_per_token=2, hidden_dim=256, max_num_tokens=16)
    fn = _entry_point()
    inp = make_rank_inputs(cfg, torch.Generator().manual_seed(5), num_tokens=16)
    x, indices = inp.x.to(device), as_index_tensor(inp.indices, device)
    got = _outputs(cfg, device)
    rc, msg = _call(fn, cfg, got[0], got[1], None, x, None, indices, None, None)
    assert rc == 0, msg
    torch.cuda.synchronize()
    assert int(got[0].sum()) == 16 * cfg.experts_per_token
    bound_m = torch.tensor([5], dtype=torch.int32, device=device)
    rc, msg = _call(fn, cfg, got[0], got[1], None, x, None, indices, bound_m, None)
    assert rc == 0, msg
    torch.cuda.synchronize()
    assert int(got[0].sum()) == 5 * cfg.experts_per_token


def test_sizes_beyond_the_built_in_staging_are_rejected():
    device = torch.device("cuda", 0)
    cfg = MoEConfig(num_experts=8, experts_per_token=8, hidden_dim=8192, max_num_tokens=256)
    fn = _entry_point()
    # 256 tokens x 8 x 16 KiB = 32 MiB > 16 MiB; nothing is launched, so tiny tensors suffice.
    x = torch.zeros(1, cfg.hidden_dim, dtype=torch.bfloat16, device=device)
    indices = torch.zeros(1, 8, dtype=torch.int32, device=device)
    counts, out_x, _ = _outputs(MoEConfig(8, 8, 8192, 1), device)
    rc, msg = _call(fn, cfg, counts, out_x, None, x, None, indices, None, None, num_tokens=256)
    assert rc == -2 and "exceeds the built-in staging" in msg
    big = MoEConfig(num_experts=2048, experts_per_token=2, hidden_dim=64, max_num_tokens=1)
    rc, msg = _call(fn, big, counts, out_x, None, x, None, indices, None, None, num_tokens=1)
    assert rc == -2 and "1024" in msg
    bad = MoEConfig(num_experts=8, experts_per_token=2, hidden_dim=36, max_num_tokens=1)
    rc, msg = _call(fn, bad, counts, out_x, None, x, None, indices, None, None, num_tokens=1)
    assert rc == -1 and "multiple of 16" in msg
