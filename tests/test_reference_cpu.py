"""CPU tests of the pure-torch oracle over gloo (world_size 2 and 4)."""

import pytest
import torch

from pplx_kernels_b200.ops.reference import (
    ReferenceAllToAll,
    simulate_combine,
    simulate_dispatch,
)
from pplx_kernels_b200.utils.testing import (
    MoEConfig,
    ProcessGroupInfo,
    make_rank_inputs,
    parallel_launch,
)


def _world_inputs(cfg: MoEConfig, num_dp: int, dp_size: int, seed: int, **kw):
    gen = torch.Generator().manual_seed(seed)
    per_group = [make_rank_inputs(cfg, gen, **kw) for _ in range(num_dp)]
    return [per_group[r // dp_size] for r in range(num_dp * dp_size)]


def _oracle_worker(pgi: ProcessGroupInfo, cfg: MoEConfig, dp_size: int, identity: bool) -> None:
    world, rank = pgi.world_size, pgi.rank
    num_dp = world // dp_size
    inputs = _world_inputs(cfg, num_dp, dp_size, seed=7, softmax_weights=identity,
                           num_tokens=cfg.max_num_tokens if identity else None)
    mine = inputs[rank]
    nle = -(-cfg.num_experts // world)
    ata = ReferenceAllToAll(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token, rank,
                            world, dp_size, cfg.hidden_dim, cfg.hidden_dim_bytes,
                            cfg.hidden_dim_scale_bytes)
    counts = torch.empty(nle, dtype=torch.int32)
    expert_x = torch.zeros(nle, cfg.max_num_tokens * num_dp, cfg.hidden_dim, dtype=cfg.in_dtype)
    expert_scale = None
    if cfg.hidden_dim_scale:
        expert_scale = torch.zeros(nle, expert_x.size(1), cfg.hidden_dim_scale)
    bound_m = torch.tensor([mine.num_tokens], dtype=torch.int32)
    ata.dispatch(counts, expert_x, expert_scale, mine.x, mine.x_scale, mine.indices, bound_m)

    expected = simulate_dispatch(inputs, cfg.num_experts, dp_size)[rank]
    assert counts.tolist() == expected.counts()
    for le in range(nle):
        want = sorted(tuple(inputs[s].x[i].float().tolist()) for s, i, _ in expected.rows[le])
        got = sorted(tuple(expert_x[le, j].float().tolist()) for j in range(counts[le]))
        assert want == got
        if expert_scale is not None:
            want_s = sorted(tuple(inputs[s].x_scale[i].tolist()) for s, i, _ in expected.rows[le])
            got_s = sorted(tuple(expert_scale[le, j].tolist()) for j in range(counts[le]))
            assert want_s == got_s

    scale = 1.0 if identity else 1.5
    expert_y = (expert_x.float() * scale).to(cfg.out_dtype)
    out = torch.full((cfg.max_num_tokens, cfg.hidden_dim), float("nan"), dtype=cfg.out_dtype)
    ata.combine(out, mine.indices, mine.weights, expert_y, bound_m)
    want_out = simulate_combine(
        inputs, lambda e, row: (row.float() * scale).to(cfg.out_dtype), cfg.out_dtype, rank)
    torch.testing.assert_close(out[: mine.num_tokens], want_out)
    assert torch.isnan(out[mine.num_tokens:].float()).all()
    if identity:
        # softmax weights sum to one: combine(dispatch(x)) == x
        torch.testing.assert_close(out[: mine.num_tokens], mine.x.to(cfg.out_dtype),
                                   rtol=1e-5, atol=1e-5)


def test_oracle_identity_world2():
    # 8 experts (4 per rank), top-2, 16 tokens per rank, hidden 128 fp32, softmax weights.
    cfg = MoEConfig(num_experts=8, experts_per_token=2, hidden_dim=128, max_num_tokens=16,
                    in_dtype=torch.float32, out_dtype=torch.float32)
    parallel_launch(2, _oracle_worker, cfg, 1, True, use_cuda=False)


def test_oracle_uneven_expert_count_world4():
    # 10 experts over 4 ranks: blocks of 3, the last rank owns one real expert.
    cfg = MoEConfig(num_experts=10, experts_per_token=3, hidden_dim=64, max_num_tokens=9)
    parallel_launch(4, _oracle_worker, cfg, 1, False, use_cuda=False)


def test_oracle_dp_groups_world4_bf16():
    cfg = MoEConfig(num_experts=8, experts_per_token=3, hidden_dim=64, max_num_tokens=10)
    parallel_launch(4, _oracle_worker, cfg, 2, False, use_cuda=False)


def test_oracle_fp8_scales_world2():
    cfg = MoEConfig(num_experts=8, experts_per_token=3, hidden_dim=256, max_num_tokens=6,
                    in_dtype=torch.float8_e4m3fn)
    parallel_launch(2, _oracle_worker, cfg, 1, False, use_cuda=False)


def test_simulate_dispatch_counts_rows_once():
    cfg = MoEConfig(num_experts=8, experts_per_token=3, hidden_dim=16, max_num_tokens=9)
    inputs = _world_inputs(cfg, 2, 2, seed=1)
    expected = simulate_dispatch(inputs, cfg.num_experts, dp_size=2)
    total = sum(sum(e.counts()) for e in expected)
    # every (group, token, k) appears exactly once although each group has two ranks
    assert total == sum(inputs[g * 2].num_tokens for g in range(2)) * cfg.experts_per_token
    seen = set()
    for e in expected:
        for rows in e.rows:
            for src, i, k in rows:
                assert (src // 2, i, k) not in seen
                assert i % 2 == src % 2
                seen.add((src // 2, i, k))


def _env_worker(pgi: ProcessGroupInfo, expect_world: int) -> None:
    import torch.distributed as dist

    assert pgi.world_size == expect_world and pgi.world_local_size == expect_world
    assert pgi.rank == pgi.node_rank * pgi.world_local_size + pgi.local_rank
    t = torch.tensor([float(pgi.rank)])
    dist.all_reduce(t)
    assert t.item() == sum(range(expect_world))


def test_launch_from_environment_variables(monkeypatch):
    from pplx_kernels_b200.utils.testing import (
        free_port,
        launch_env_present,
        parallel_launch_from_env,
    )

    for k in ("WORLD_SIZE", "WORLD_LOCAL_SIZE", "NODE_RANK", "MASTER_ADDR", "MASTER_PORT"):
        monkeypatch.delenv(k, raising=False)
    assert not launch_env_present()
    monkeypatch.setenv("WORLD_SIZE", "2")
    monkeypatch.setenv("WORLD_LOCAL_SIZE", "2")
    monkeypatch.setenv("NODE_RANK", "0")
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", str(free_port()))
    assert launch_env_present()
    parallel_launch_from_env(_env_worker, 2, use_cuda=False)


def test_simulated_world_invariants_over_random_shapes():
    """Property check of the single-process oracle over random worlds, DP sizes, expert counts
    (even and uneven) and token counts (including none): every (group, token, k) is delivered
    exactly once, to the rank and slot that own the expert, by the rank of the group whose turn
    it is; and with weights that sum to one an identity expert gives the tokens back."""
    hypothesis = pytest.importorskip("hypothesis")
    st = hypothesis.strategies

    @hypothesis.settings(max_examples=40, deadline=None)
    @hypothesis.given(world=st.sampled_from([1, 2, 4, 8]), dp_pow=st.integers(0, 3),
                      experts=st.integers(1, 24), topk=st.integers(1, 4),
                      tokens=st.integers(0, 9), seed=st.integers(0, 10_000))
    def check(world, dp_pow, experts, topk, tokens, seed):
        dp_size = min(world, 1 << dp_pow)
        topk = min(topk, experts)
        cfg = MoEConfig(num_experts=experts, experts_per_token=topk, hidden_dim=8,
                        max_num_tokens=max(tokens, 1), in_dtype=torch.float32,
                        out_dtype=torch.float32)
        inputs = _world_inputs(cfg, world // dp_size, dp_size, seed=seed, num_tokens=tokens,
                               softmax_weights=True)
        expected = simulate_dispatch(inputs, experts, dp_size)
        nle = -(-experts // world)
        seen = set()
        for dst, e in enumerate(expected):
            assert len(e.rows) == nle
            for le, rows in enumerate(e.rows):
                for src, i, k in rows:
                    g = int(inputs[src].indices[i, k])
                    assert g // nle == dst and g % nle == le
                    assert i % dp_size == src % dp_size
                    assert (src // dp_size, i, k) not in seen
                    seen.add((src // dp_size, i, k))
        assert len(seen) == (world // dp_size) * tokens * topk
        for rank in range(world):
            out = simulate_combine(inputs, lambda e, row: row.float(), torch.float32, rank)
            torch.testing.assert_close(out, inputs[rank].x[:tokens].float(), rtol=1e-5, atol=1e-5)

    check()


def test_the_decode_sized_protocol_yields_the_oracles_rows_in_the_oracles_order():
    """Headers per (destination, source, token slot) and a row table derived from them in
    (source, slot, j) order -- the algorithm of the decode-sized dispatch kernel -- give exactly
    the per-expert row lists of the oracle, order included, for any routing, DP split, expert
    count that does not divide, and groups with fewer tokens than slots."""
    from pplx_kernels_b200.ops.reference import simulate_dispatch_by_headers

    hypothesis = pytest.importorskip("hypothesis")
    st = hypothesis.strategies

    @hypothesis.settings(max_examples=40, deadline=None)
    @hypothesis.given(world=st.sampled_from([1, 2, 4, 8]), dp_pow=st.integers(0, 3),
                      experts=st.integers(1, 24), topk=st.integers(1, 4),
                      tokens=st.integers(0, 9), slack=st.integers(0, 3),
                      seed=st.integers(0, 10_000))
    def check(world, dp_pow, experts, topk, tokens, slack, seed):
        dp_size = min(world, 1 << dp_pow)
        topk = min(topk, experts)
        max_tokens = max(tokens, 1) + slack
        cfg = MoEConfig(num_experts=experts, experts_per_token=topk, hidden_dim=8,
                        max_num_tokens=max_tokens, in_dtype=torch.float32,
                        out_dtype=torch.float32)
        inputs = _world_inputs(cfg, world // dp_size, dp_size, seed=seed, num_tokens=tokens)
        want = simulate_dispatch(inputs, experts, dp_size)
        got = simulate_dispatch_by_headers(inputs, experts, dp_size, max_tokens)
        for r in range(world):
            assert got[r].rows == want[r].rows

    check()
