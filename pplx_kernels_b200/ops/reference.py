"""Pure-torch statement of what dispatch and combine mean.

Two forms are provided:

* ``ReferenceAllToAll`` has the signature of ``AllToAll`` and runs on any
  device over ``torch.distributed`` (gloo on CPU), one process per rank.  It is
  the oracle for the host-side logic and the CPU baseline for tiny shapes.
* ``simulate_dispatch`` / ``simulate_combine`` compute, inside one process, what
  every rank of a world must end up with.  GPU tests compare the kernels
  against them.

Semantics restated from the reference's kernels (intranode_dispatch.cu:97-275,
intranode_combine.cu:77-169): ranks ``[g*dp_size, (g+1)*dp_size)`` hold the same
tokens; token ``i`` of a group is sent by the rank with ``i % dp_size`` equal to
its position in the group; expert ``e`` lives on rank ``e // num_local_experts``;
each rank receives, per local expert, the rows routed to it (in any order) and
their count; combine returns every expert output row to all ranks of the
token's group and reduces ``sum_k weights[i, k] * y`` in float32, in ``k`` order,
with one final cast.  Rows at or beyond ``bound_m`` are not touched.
"""

from __future__ import annotations

import dataclasses
from collections.abc import Sequence

import torch
import torch.distributed as dist


def _num_tokens(indices: torch.Tensor, bound_m: torch.Tensor | None) -> int:
    m = indices.size(0)
    if bound_m is not None:
        m = min(m, int(bound_m.view(-1)[0].item()))
    return m


def _as_bytes(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8)


# --------------------------------------------------------------------------------
# Single-process simulation of a whole world
# --------------------------------------------------------------------------------


@dataclasses.dataclass
class RankInputs:
    """What one rank passes to dispatch (CPU or GPU tensors)."""

    x: torch.Tensor  # [m, hidden]
    x_scale: torch.Tensor | None  # [m, hidden_scale] float32
    indices: torch.Tensor  # [m, topk]
    weights: torch.Tensor  # [m, topk] float32
    num_tokens: int  # bound_m


@dataclasses.dataclass
class ExpectedDispatch:
    """Rows every local expert of one rank must receive, as (source rank, token, k)."""

    rows: list[list[tuple[int, int, int]]]  # [num_local_experts] -> list of sources

    def counts(self) -> list[int]:
        return [len(r) for r in self.rows]


def simulate_dispatch(
    inputs: Sequence[RankInputs], num_experts: int, dp_size: int
) -> list[ExpectedDispatch]:
    """``inputs[r]`` is rank r's data; ranks of one DP group must hold equal data."""
    from ..parallel.placement import EPLayout

    world = len(inputs)
    layout = EPLayout(num_experts, world, dp_size)  # who owns an expert, who sends a token
    out = [ExpectedDispatch([[] for _ in range(layout.num_local_experts)]) for _ in range(world)]
    for src in range(world):
        group = layout.dp_group(src)
        idx = inputs[src].indices.cpu().to(torch.int64)
        for i in range(inputs[src].num_tokens):
            if layout.sender_of(group, i) != src:
                continue
            for k in range(idx.size(1)):
                e = int(idx[i, k])
                out[layout.owner(e)].rows[layout.local_index(e)].append((src, i, k))
    return out


def simulate_dispatch_by_headers(
    inputs: Sequence[RankInputs], num_experts: int, dp_size: int, max_num_tokens: int
) -> list[ExpectedDispatch]:
    """The decode-sized dispatch (csrc/kernels/dispatch_tiny.cu) restated step by step: every
    sender writes, for every destination and every one of its token slots (filled or not), a
    header ``[(k, local expert), ...]``; every receiver walks the headers in (source, token slot,
    j) order and gives entry number n of a local expert output row n.  The result has to be the
    very lists that ``simulate_dispatch`` builds, in the same order: the kernel's row order is
    deterministic, unlike the general kernel's."""
    from ..parallel.placement import EPLayout

    world = len(inputs)
    layout = EPLayout(num_experts, world, dp_size)
    slots_per_sender = -(-max_num_tokens // dp_size)
    # headers[dst][src][slot] -> [(k, local expert)]
    headers = [[[[] for _ in range(slots_per_sender)] for _ in range(world)] for _ in range(world)]
    for src in range(world):
        idx = inputs[src].indices.cpu().to(torch.int64)
        for o in range(slots_per_sender):
            i = o * dp_size + src % dp_size
            if i >= inputs[src].num_tokens:
                continue  # the slot's headers stay empty, but they are written
            for k in range(idx.size(1)):
                e = int(idx[i, k])
                headers[layout.owner(e)][src][o].append((k, layout.local_index(e)))
    out = [ExpectedDispatch([[] for _ in range(layout.num_local_experts)]) for _ in range(world)]
    for dst in range(world):
        for src in range(world):
            for o in range(slots_per_sender):
                for k, le in headers[dst][src][o]:
                    out[dst].rows[le].append((src, o * dp_size + src % dp_size, k))
    return out


def simulate_combine(
    inputs: Sequence[RankInputs],
    expert_fn,
    out_dtype: torch.dtype,
    rank: int,
) -> torch.Tensor:
    """Expected ``out_tokens[:num_tokens]`` of ``rank`` when every expert applies
    ``expert_fn(global_expert, x_row_float32) -> y_row`` (already in the dtype the
    expert output has on the wire)."""
    inp = inputs[rank]
    m = inp.num_tokens
    x = inp.x.cpu()
    idx = inp.indices.cpu().to(torch.int64)
    w = inp.weights.cpu().to(torch.float32)
    hidden = x.size(1)
    acc = torch.zeros(m, hidden, dtype=torch.float32)
    for i in range(m):
        for k in range(idx.size(1)):
            y = expert_fn(int(idx[i, k]), x[i])
            acc[i] = torch.addcmul(acc[i], y.to(torch.float32), w[i, k])
    return acc.to(out_dtype)


# --------------------------------------------------------------------------------
# Multi-process oracle with the AllToAll signature
# --------------------------------------------------------------------------------


class ReferenceAllToAll:
    """Dispatch/combine over ``torch.distributed`` collectives, no custom kernels."""

    def __init__(
        self,
        max_num_tokens: int,
        num_experts: int,
        experts_per_token: int,
        rank: int,
        world_size: int,
        dp_size: int,
        hidden_dim: int,
        hidden_dim_bytes: int,
        hidden_dim_scale_bytes: int,
        group: dist.ProcessGroup | None = None,
    ) -> None:
        assert world_size % dp_size == 0
        self.max_num_tokens = max_num_tokens
        self.num_experts = num_experts
        self.topk = experts_per_token
        self.rank = rank
        self.world = world_size
        self.dp_size = dp_size
        self.num_dp_groups = world_size // dp_size
        self.nle = -(-num_experts // world_size)
        self.hidden_dim = hidden_dim
        self.hidden_bytes = hidden_dim_bytes
        self.scale_bytes = hidden_dim_scale_bytes
        self.group = group
        self._has_scales = hidden_dim_scale_bytes > 0
        # (source rank, token, k) of every received row, per local expert
        self._row_src: list[list[tuple[int, int, int]]] | None = None

    # Kept for signature parity with AllToAll.
    @classmethod
    def intranode(cls, *args, group_name: str = "default", **kwargs) -> "ReferenceAllToAll":
        return cls(*args, **kwargs)

    @classmethod
    def internode(cls, *args, **kwargs) -> "ReferenceAllToAll":
        return cls(*args, **kwargs)

    def destroy(self) -> None:
        self._row_src = None

    def _exchange(self, send: list[torch.Tensor], row_bytes: int) -> list[torch.Tensor]:
        """``send[d]`` is a uint8 [n_d, row_bytes] tensor for rank d; returns what came."""
        device = send[0].device
        counts = torch.tensor([t.size(0) for t in send], dtype=torch.int64, device=device)
        got = torch.empty_like(counts)
        if self.world > 1:
            dist.all_to_all_single(got, counts, group=self.group)
        else:
            got.copy_(counts)
        in_splits = [int(c) * row_bytes for c in counts.tolist()]
        out_splits = [int(c) * row_bytes for c in got.tolist()]
        flat_in = torch.cat([t.reshape(-1) for t in send]) if sum(in_splits) else torch.empty(
            0, dtype=torch.uint8, device=device)
        flat_out = torch.empty(sum(out_splits), dtype=torch.uint8, device=device)
        if self.world > 1:
            dist.all_to_all_single(flat_out, flat_in, out_splits, in_splits, group=self.group)
        else:
            flat_out.copy_(flat_in)
        parts = torch.split(flat_out, out_splits)
        return [p.view(-1, row_bytes) for p in parts]

    def dispatch(
        self,
        out_expert_num_tokens: torch.Tensor,
        out_expert_x: torch.Tensor,
        out_expert_x_scale: torch.Tensor | None,
        dp_x: torch.Tensor,
        dp_x_scale: torch.Tensor | None,
        indices: torch.Tensor,
        bound_m: torch.Tensor | None,
        do_send: bool = True,
        do_recv: bool = True,
    ) -> None:
        assert do_send and do_recv, "the oracle has no split mode"
        assert self._has_scales == (dp_x_scale is not None) == (out_expert_x_scale is not None)
        device = dp_x.device
        m = _num_tokens(indices, bound_m)
        idx = indices.cpu().to(torch.int64)
        xb = _as_bytes(dp_x).view(dp_x.size(0), self.hidden_bytes)
        sb = None
        if dp_x_scale is not None:
            sb = _as_bytes(dp_x_scale.to(torch.float32)).view(dp_x.size(0), self.scale_bytes)
        row_bytes = self.hidden_bytes + self.scale_bytes + 12
        per_dst: list[list[torch.Tensor]] = [[] for _ in range(self.world)]
        dp_rank = self.rank % self.dp_size
        for i in range(dp_rank, m, self.dp_size):
            for k in range(self.topk):
                e = int(idx[i, k])
                meta = torch.tensor([i, k, e % self.nle], dtype=torch.int32, device=device)
                pieces = [xb[i]]
                if sb is not None:
                    pieces.append(sb[i])
                pieces.append(meta.view(torch.uint8))
                per_dst[e // self.nle].append(torch.cat(pieces))
        send = [
            torch.stack(rows) if rows else torch.empty(0, row_bytes, dtype=torch.uint8, device=device)
            for rows in per_dst
        ]
        got = self._exchange(send, row_bytes)

        self._row_src = [[] for _ in range(self.nle)]
        out_xb = out_expert_x.view(torch.uint8).view(self.nle, out_expert_x.size(1), self.hidden_bytes)
        for src, rows in enumerate(got):
            for r in range(rows.size(0)):
                row = rows[r]
                meta = row[self.hidden_bytes + self.scale_bytes:].contiguous().view(torch.int32)
                i, k, le = (int(v) for v in meta.tolist())
                pos = len(self._row_src[le])
                out_xb[le, pos] = row[: self.hidden_bytes]
                if out_expert_x_scale is not None:
                    out_expert_x_scale[le, pos] = (
                        row[self.hidden_bytes : self.hidden_bytes + self.scale_bytes]
                        .contiguous()
                        .view(torch.float32)
                    )
                self._row_src[le].append((src, i, k))
        out_expert_num_tokens.copy_(
            torch.tensor([len(r) for r in self._row_src], dtype=torch.int32, device=device)
        )

    def combine(
        self,
        out_tokens: torch.Tensor,
        indices: torch.Tensor,
        weights: torch.Tensor,
        expert_y: torch.Tensor,
        bound_m: torch.Tensor | None,
        do_send: bool = True,
        do_recv: bool = True,
    ) -> None:
        assert do_send and do_recv, "the oracle has no split mode"
        assert self._row_src is not None, "combine must follow a dispatch"
        device = expert_y.device
        m = _num_tokens(indices, bound_m)
        y_bytes = self.hidden_dim * expert_y.element_size()
        row_bytes = y_bytes + 8
        per_dst: list[list[torch.Tensor]] = [[] for _ in range(self.world)]
        for le, rows in enumerate(self._row_src):
            for pos, (src, i, k) in enumerate(rows):
                meta = torch.tensor([i, k], dtype=torch.int32, device=device).view(torch.uint8)
                payload = torch.cat([_as_bytes(expert_y[le, pos]), meta])
                group_first = (src // self.dp_size) * self.dp_size
                for r in range(self.dp_size):
                    per_dst[group_first + r].append(payload)
        send = [
            torch.stack(rows) if rows else torch.empty(0, row_bytes, dtype=torch.uint8, device=device)
            for rows in per_dst
        ]
        got = self._exchange(send, row_bytes)

        stage = torch.zeros(m, self.topk, self.hidden_dim, dtype=torch.float32, device=device)
        for rows in got:
            for r in range(rows.size(0)):
                row = rows[r]
                i, k = (int(v) for v in row[y_bytes:].contiguous().view(torch.int32).tolist())
                stage[i, k] = row[:y_bytes].contiguous().view(expert_y.dtype).to(torch.float32)
        acc = torch.zeros(m, self.hidden_dim, dtype=torch.float32, device=device)
        w = weights.to(torch.float32)
        for k in range(self.topk):
            acc = torch.addcmul(acc, stage[:, k], w[:m, k : k + 1])
        out_tokens[:m] = acc.to(out_tokens.dtype)
        self._row_src = None
