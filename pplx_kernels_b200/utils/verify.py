"""Verification of dispatch / combine results against the pure-PyTorch oracle (used by the
GPU tests, the smoke run and the benchmarks that check their output before timing).

Follows the reference's checks (tests/test_all_to_all.py:195-286): per-expert
counts equal the expectation computed from the routing tables, received rows
equal the expected rows as a multiset (row order is unspecified), and combine
into a NaN-prefilled buffer matches ``sum_k w_k * y_k``.  Stronger than the
reference in one point: payload and scales are compared as one joined row, so a
scale row attached to the wrong token is caught.
"""

from __future__ import annotations

import torch

import pplx_kernels_b200 as pk
from pplx_kernels_b200.ops.reference import RankInputs, simulate_combine, simulate_dispatch
from pplx_kernels_b200.utils.testing import MoEConfig, as_index_tensor, make_rank_inputs

EXPERT_GAIN = 1.5


def world_inputs(cfg: MoEConfig, world: int, dp_size: int, seed: int, **kw) -> list[RankInputs]:
    """`num_tokens` may be a list with one entry per DP group."""
    gen = torch.Generator().manual_seed(seed)
    counts = kw.pop("num_tokens", None)
    groups = world // dp_size
    if not isinstance(counts, (list, tuple)):
        counts = [counts] * groups
    assert len(counts) == groups
    per_group = [make_rank_inputs(cfg, gen, num_tokens=counts[g], **kw) for g in range(groups)]
    return [per_group[r // dp_size] for r in range(world)]


class RankBuffers:
    """Device tensors one rank passes to dispatch and combine."""

    def __init__(self, cfg: MoEConfig, world: int, dp_size: int, inp: RankInputs,
                 device: torch.device, strided_scale: bool = False,
                 use_bound_m: bool = True) -> None:
        nle = -(-cfg.num_experts // world)
        rows = cfg.max_num_tokens * (world // dp_size)
        self.cfg = cfg
        self.num_tokens = inp.num_tokens
        self.counts = torch.full((nle,), -1, dtype=torch.int32, device=device)
        self.expert_x = torch.zeros(nle, rows, cfg.hidden_dim, device=device).to(cfg.in_dtype)
        self.expert_scale = None
        self.x_scale = None
        if cfg.hidden_dim_scale:
            if strided_scale:
                # [nle, scale, rows] storage viewed as [nle, rows, scale]: no unit stride
                # in the last dimension, as a caller with a transposed scale layout has.
                base = torch.zeros(nle, cfg.hidden_dim_scale, rows, device=device)
                self.expert_scale = base.transpose(1, 2)
                xs = inp.x_scale.to(device).t().contiguous().t()
            else:
                self.expert_scale = torch.zeros(nle, rows, cfg.hidden_dim_scale, device=device)
                xs = inp.x_scale.to(device)
            self.x_scale = xs
        if use_bound_m:
            # The tensors hold max_num_tokens rows; only the first bound_m are valid and
            # the rest carry expert ids that would trip the bounds checks if read.
            pad = cfg.max_num_tokens - inp.num_tokens
            self.x = torch.cat([inp.x, torch.zeros(pad, cfg.hidden_dim).to(cfg.in_dtype)]).to(device)
            junk = torch.full((pad, cfg.experts_per_token), 0x7FFFFFF0, dtype=torch.int32)
            self.indices = as_index_tensor(torch.cat([inp.indices, junk]), device)
            self.weights = torch.cat([inp.weights, torch.zeros(pad, cfg.experts_per_token)]).to(device)
            if self.x_scale is not None:
                extra = torch.zeros(pad, cfg.hidden_dim_scale, device=device)
                if strided_scale:
                    self.x_scale = torch.cat([self.x_scale, extra]).t().contiguous().t()
                else:
                    self.x_scale = torch.cat([self.x_scale, extra])
            self.bound_m = torch.tensor([inp.num_tokens], dtype=torch.int32,
                                        device=device).view(torch.uint32)
        else:
            m = inp.num_tokens
            self.x = inp.x[:m].to(device)
            self.indices = as_index_tensor(inp.indices[:m], device)
            self.weights = inp.weights[:m].to(device)
            if self.x_scale is not None:
                self.x_scale = self.x_scale[:m]
            self.bound_m = None
        self.out = torch.full((cfg.max_num_tokens, cfg.hidden_dim), float("nan"),
                              device=device).to(cfg.out_dtype)
        self.expert_y: torch.Tensor | None = None

    def make_expert_y(self, y_dtype: torch.dtype | None = None) -> torch.Tensor:
        y_dtype = y_dtype or self.cfg.out_dtype
        self.expert_y = (self.expert_x.to(torch.float32) * EXPERT_GAIN).to(y_dtype)
        return self.expert_y


def _joined_rows(x: torch.Tensor, scale: torch.Tensor | None) -> torch.Tensor:
    rows = x.contiguous().view(torch.uint8).view(x.size(0), -1).to(torch.int64)
    if scale is not None:
        s = scale.contiguous().to(torch.float32).view(torch.uint8).view(x.size(0), -1)
        rows = torch.cat([rows, s.to(torch.int64)], dim=1)
    return rows


def _sorted_rows(rows: torch.Tensor) -> torch.Tensor:
    if rows.size(0) == 0:
        return rows
    gen = torch.Generator().manual_seed(99)
    w = torch.randint(1, 1 << 20, (rows.size(1),), generator=gen, dtype=torch.int64)
    key = (rows * w).sum(dim=1)
    return rows[torch.argsort(key, stable=True)]


def verify_dispatch(cfg: MoEConfig, inputs: list[RankInputs], dp_size: int, rank: int,
                    buf: RankBuffers) -> None:
    world = len(inputs)
    expected = simulate_dispatch(inputs, cfg.num_experts, dp_size)[rank]
    counts = buf.counts.cpu().tolist()
    assert counts == expected.counts(), f"rank {rank}: counts {counts} != {expected.counts()}"
    expert_x = buf.expert_x.cpu()
    expert_scale = buf.expert_scale.cpu() if buf.expert_scale is not None else None
    for le, rows in enumerate(expected.rows):
        n = len(rows)
        if n == 0:
            continue
        want_x = torch.stack([inputs[s].x[i] for s, i, _ in rows])
        want_s = None
        got_s = None
        if expert_scale is not None:
            want_s = torch.stack([inputs[s].x_scale[i] for s, i, _ in rows])
            got_s = expert_scale[le, :n]
        want = _sorted_rows(_joined_rows(want_x, want_s))
        got = _sorted_rows(_joined_rows(expert_x[le, :n], got_s))
        assert torch.equal(want, got), f"rank {rank} expert {le}: received rows differ"
    del world


def verify_combine(cfg: MoEConfig, inputs: list[RankInputs], rank: int, buf: RankBuffers,
                   y_dtype: torch.dtype | None = None) -> None:
    y_dtype = y_dtype or cfg.out_dtype
    want = simulate_combine(
        inputs, lambda e, row: (row.to(torch.float32) * EXPERT_GAIN).to(y_dtype),
        cfg.out_dtype, rank)
    m = inputs[rank].num_tokens
    got = buf.out.cpu()
    torch.testing.assert_close(got[:m], want)
    assert torch.isnan(got[m:].to(torch.float32)).all(), "rows beyond bound_m were written"


def run_local_world(cfg: MoEConfig, world: int, dp_size: int, seed: int = 0,
                    iterations: int = 1, split: bool = False, use_bound_m: bool = True,
                    strided_scale: bool = False, y_dtype: torch.dtype | None = None,
                    max_blocks: int = 0, **input_kw) -> None:
    """All ranks of a world on GPU 0, driven through the group launches."""
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    ranks = pk.AllToAll.local_world(
        cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token, world, dp_size,
        cfg.hidden_dim, cfg.hidden_dim_bytes, cfg.hidden_dim_scale_bytes)
    try:
        for r in ranks:
            r.set_debug_checks(True)
            r.set_timeout_ms(3000)
            if max_blocks:
                r.set_max_blocks(max_blocks)
        for it in range(iterations):
            inputs = world_inputs(cfg, world, dp_size, seed + 17 * it, **input_kw)
            bufs = [RankBuffers(cfg, world, dp_size, inputs[r], device, strided_scale, use_bound_m)
                    for r in range(world)]
            d_args = ([b.counts for b in bufs], [b.expert_x for b in bufs],
                      [b.expert_scale for b in bufs], [b.x for b in bufs],
                      [b.x_scale for b in bufs], [b.indices for b in bufs],
                      [b.bound_m for b in bufs])
            if split:
                pk.dispatch_group(ranks, *d_args, do_send=True, do_recv=False)
                pk.dispatch_group(ranks, *d_args, do_send=False, do_recv=True)
            else:
                pk.dispatch_group(ranks, *d_args)
            torch.cuda.synchronize()
            for r in range(world):
                ranks[r].check_status()
                verify_dispatch(cfg, inputs, dp_size, r, bufs[r])
            c_args = ([b.out for b in bufs], [b.indices for b in bufs],
                      [b.weights for b in bufs], [b.make_expert_y(y_dtype) for b in bufs],
                      [b.bound_m for b in bufs])
            if split:
                pk.combine_group(ranks, *c_args, do_send=True, do_recv=False)
                pk.combine_group(ranks, *c_args, do_send=False, do_recv=True)
            else:
                pk.combine_group(ranks, *c_args)
            torch.cuda.synchronize()
            for r in range(world):
                ranks[r].check_status()
                verify_combine(cfg, inputs, r, bufs[r], y_dtype)
    finally:
        for r in ranks:
            r.destroy()
