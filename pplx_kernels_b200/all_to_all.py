"""Python face of the dispatch/combine all-to-all.

Role parity: src/pplx_kernels/all_to_all.py:11-164 of the reference.  The class
name, the two constructors, the ``dispatch``/``combine``/``destroy`` methods and
all argument names and orders are the same, so code written against the
reference runs unchanged.  Additions: ``check_status`` (a wait that ran out is
reported instead of hanging), tunables, and ``local_world`` / ``dispatch_group``
/ ``combine_group`` which run several ranks on one GPU inside a single
cooperative launch.  The reference's requirement of more than one DP group is
dropped: ``world_size == dp_size`` (including a single GPU) is accepted.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from typing import Any

import torch

from .ops import _ops


def _resolve_group_name(group_name: str) -> str:
    """Returns a name that the C++ side can resolve to a ProcessGroup."""
    c10d = torch._C._distributed_c10d
    try:
        c10d._resolve_process_group(group_name)
        return group_name
    except Exception:
        pass
    import torch.distributed as dist

    if not dist.is_initialized():
        raise RuntimeError(
            f"process group {group_name!r} is not registered and torch.distributed is not initialised"
        )
    world = dist.group.WORLD
    try:
        c10d._register_process_group(group_name, world)
        return group_name
    except Exception:
        return world.group_name


class AllToAll:
    def __init__(
        self,
        ptr: Any,
        combine_fn: Callable,
        dispatch_fn: Callable,
        has_scales: bool,
    ) -> None:
        self._ptr = ptr
        self._combine_fn = combine_fn
        self._dispatch_fn = dispatch_fn
        self._has_scales = has_scales

    def __del__(self) -> None:
        try:
            self.destroy()
        except Exception:
            pass

    # ------------------------------------------------------------ operations --

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
        assert self._ptr is not None
        if self._has_scales:
            assert out_expert_x_scale is not None
            assert dp_x_scale is not None
        else:
            assert out_expert_x_scale is None
            assert dp_x_scale is None
        self._dispatch_fn(
            self._ptr,
            out_expert_num_tokens,
            out_expert_x,
            out_expert_x_scale,
            dp_x,
            dp_x_scale,
            indices,
            bound_m,
            do_send,
            do_recv,
        )

    def dispatch_quant(
        self,
        out_expert_num_tokens: torch.Tensor,
        out_expert_x: torch.Tensor,
        out_expert_x_scale: torch.Tensor,
        dp_x: torch.Tensor,
        indices: torch.Tensor,
        bound_m: torch.Tensor | None,
        do_send: bool = True,
        do_recv: bool = True,
    ) -> None:
        """Dispatch of bf16 tokens with the fp8 block quantisation fused into the send.

        ``dp_x`` is ``[m, hidden]`` bfloat16; experts receive ``float8_e4m3fn`` rows in
        ``out_expert_x`` and one fp32 scale per 128 columns in ``out_expert_x_scale``
        (``x ~= q * scale``, ``scale = max(amax, 1e-4) / 448``).  The object must have been
        created with ``hidden_dim_bytes = hidden`` and
        ``hidden_dim_scale_bytes = ceil(hidden / 128) * 4``.
        """
        assert self._ptr is not None and self._has_scales
        _ops.all_to_all_dispatch_quant(
            self._ptr, out_expert_num_tokens, out_expert_x, out_expert_x_scale, dp_x, indices,
            bound_m, do_send, do_recv)

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
        """``out_tokens`` may also be a pinned host tensor: the reduction then writes the
        tokens to host memory itself (valid once the stream has been synchronised) and the
        separate device-to-host copy of small decode batches goes away.  ``weights`` and
        ``indices`` may be pinned host tensors as well."""
        assert self._ptr is not None
        self._combine_fn(
            self._ptr,
            out_tokens,
            indices,
            weights,
            expert_y,
            bound_m,
            do_send,
            do_recv,
        )

    def destroy(self) -> None:
        if self._ptr is not None:
            _ops.all_to_all_destroy(self._ptr)
            self._ptr = None

    # ---------------------------------------------------- status and tunables --

    def status(self) -> dict[str, int]:
        """Failure record of this object; ``code == 0`` means healthy.  Synchronises."""
        keys = ("code", "phase", "peer", "expected", "observed", "block", "rank", "count")
        return dict(zip(keys, _ops.all_to_all_status(self._ptr), strict=True))

    def peek_status(self) -> dict[str, int]:
        """The host-visible mirror of the failure record.  Does not touch the device, so it
        can be polled by a watchdog while kernels are still inside their waits."""
        keys = ("code", "phase", "peer", "expected", "observed", "block", "rank", "count")
        return dict(zip(keys, _ops.all_to_all_peek_status(self._ptr), strict=True))

    def check_status(self) -> None:
        """Raises RuntimeError if a device-side wait ran out or a bounds check failed.

        Reads the host-visible mirror: synchronise the stream first to cover the kernels
        launched so far.  Once a failure is recorded the object refuses further
        ``dispatch`` / ``combine`` calls until it is destroyed or ``reset()``.
        """
        _ops.all_to_all_check_status(self._ptr)

    def reset(self) -> None:
        """Clears this rank's flags, counters, staging and failure record.

        Collective by contract: after a failure every rank calls ``reset()`` once none of the
        object's kernels is in flight on any rank, and the ranks meet at a barrier of the
        caller's (``torch.distributed.barrier()`` will do) before the next ``dispatch``.
        """
        _ops.all_to_all_reset(self._ptr)

    def verify_canaries(self) -> None:
        """Raises if a guard word behind one of the arena's regions was overwritten (synchronises)."""
        _ops.all_to_all_verify_canaries(self._ptr)

    def set_timeout_ms(self, ms: float) -> None:
        _ops.all_to_all_set_timeout_ms(self._ptr, float(ms))

    def set_debug_checks(self, on: bool) -> None:
        _ops.all_to_all_set_debug_checks(self._ptr, bool(on))

    def set_power_of_two_scales(self, on: bool) -> None:
        """The quantising sends (``dispatch_quant``, ``fused_dispatch(quantize=True)``) round each
        scale up to a power of two, and ``fused_up_fp8`` / ``fused_down_fp8`` let the tensor cores
        apply the scales (``kind::mxf8f6f4.block_scale``) instead of the CUDA cores.  The weight
        scales passed to those calls must then be powers of two as well
        (``quantize_weight_blocks(..., pow2=True)``)."""
        _ops.all_to_all_set_quant_pow2(self._ptr, bool(on))

    def set_max_blocks(self, n: int) -> None:
        _ops.all_to_all_set_max_blocks(self._ptr, int(n))

    def set_combine_units(self, units: int) -> None:
        """No effect, kept for callers of earlier versions: arrival of expert outputs is
        counted in columns, so senders need not agree on a unit."""
        _ops.all_to_all_set_combine_units(self._ptr, int(units))

    def fused_dispatch(self, dp_x: torch.Tensor, indices: torch.Tensor,
                       bound_m: torch.Tensor | None = None, quantize: bool = False) -> None:
        """Send half of the fused MoE dispatch (bf16 tokens).

        Two-hop protocol: ranks first exchange their per-expert histograms, then store
        every row at its final, expert-major position in the destination's staging, so
        that ``fused_up`` can read dense 128-row tiles by TMA.  Follow it with
        ``fused_up``, ``fused_down`` and ``combine(..., do_send=False)``.

        With ``quantize`` (object created with ``hidden_dim_bytes = hidden`` and
        ``hidden_dim_scale_bytes = ceil(hidden / 128) * 4``) the rows travel as e4m3 with one
        fp32 scale per 128 columns, converted while they are sent; follow it with
        ``fused_up_fp8`` and ``fused_down_fp8``.
        """
        _ops.moe_dispatch_send(self._ptr, dp_x, indices, bound_m, quantize)

    def fused_up_fp8(self, w13: torch.Tensor, w13_scale: torch.Tensor, h: torch.Tensor,
                     h_scale: torch.Tensor, out_expert_num_tokens: torch.Tensor | None = None,
                     status: torch.Tensor | None = None) -> None:
        """Block-scaled fp8 SwiGLU up projection that reads rows and their scales out of the
        dispatch staging arena as peers fill it; writes the re-quantised intermediate
        (``h`` e4m3, ``h_scale`` one fp32 per row and 128 columns)."""
        _ops.moe_fused_up_fp8(self._ptr, w13, w13_scale, h, h_scale, out_expert_num_tokens, status)

    def fused_down_fp8(self, h: torch.Tensor, h_scale: torch.Tensor, w2: torch.Tensor,
                       w2_scale: torch.Tensor, status: torch.Tensor | None = None) -> None:
        """Block-scaled fp8 down projection whose epilogue stores each bf16 row to its token's
        home rank(s); call before ``combine(..., do_send=False, do_recv=True)``."""
        _ops.moe_fused_down_fp8(self._ptr, h, h_scale, w2, w2_scale, status)

    def fused_up(self, w13: torch.Tensor, h: torch.Tensor,
                 out_expert_num_tokens: torch.Tensor | None = None,
                 status: torch.Tensor | None = None, expected_rows: int = 0) -> None:
        """SwiGLU up projection that reads the dispatch staging arena as peers fill it.

        Call after ``fused_dispatch``; it replaces the receive half of dispatch.  ``h[le, :n] = silu(x @ gate.T) * (x @ up.T)`` for the rows of local expert le.
        """
        _ops.moe_fused_up(self._ptr, w13, h, out_expert_num_tokens, status, expected_rows)

    def fused_down(self, h: torch.Tensor, w2: torch.Tensor,
                   status: torch.Tensor | None = None, expected_rows: int = 0) -> None:
        """Down projection whose epilogue stores each row to its token's home rank(s).

        Call before ``combine(..., do_send=False, do_recv=True)``; it replaces the send half.
        """
        _ops.moe_fused_down(self._ptr, h, w2, status, expected_rows)

    def set_trace(self, on: bool) -> None:
        """Turns the per-phase device time stamps of block 0 on or off."""
        _ops.all_to_all_set_trace(self._ptr, bool(on))

    def read_trace(self) -> dict[str, int]:
        """Last recorded %globaltimer stamps in nanoseconds, by phase name.  Synchronises."""
        t = _ops.all_to_all_read_trace(self._ptr)
        names = {
            0: "dispatch_start", 1: "dispatch_hist", 2: "dispatch_posted", 3: "dispatch_stored",
            4: "dispatch_signalled", 5: "dispatch_counts", 6: "dispatch_layout",
            7: "dispatch_copied", 8: "dispatch_end", 16: "combine_start", 17: "combine_layout",
            18: "combine_sent", 19: "combine_reduced", 20: "combine_end",
        }
        out = {name: t[i] for i, name in names.items()}
        # Per-block stamps: earliest start and latest end over the blocks that ran.
        nb = 256
        for j, key in enumerate(("dispatch_blocks", "combine_blocks")):
            starts = [v for v in t[32 + 2 * j * nb: 32 + (2 * j + 1) * nb] if v]
            ends = [v for v in t[32 + (2 * j + 1) * nb: 32 + (2 * j + 2) * nb] if v]
            if starts and ends:
                out[key + "_first_start"] = min(starts)
                out[key + "_last_start"] = max(starts)
                out[key + "_first_end"] = min(ends)
                out[key + "_last_end"] = max(ends)
        return out

    def layout(self) -> dict[str, int]:
        keys = ("num_local_experts", "num_dp_groups", "rows_per_expert", "region_slots",
                "slot_bytes", "arena_bytes", "flag_in_data", "line_slot_bytes",
                "line_combine_slot_bytes", "decode_sized_dispatch", "vmm_arena", "multicast")
        return dict(zip(keys, _ops.all_to_all_layout(self._ptr), strict=True))

    def multicast_note(self) -> str:
        """Why NVLink multicast was asked for (``PPLX_B200_MULTIMEM=1``) but is not in use;
        empty when it is in use or was not asked for."""
        return _ops.all_to_all_multicast_note(self._ptr)

    # ------------------------------------------------------------ constructors --

    @classmethod
    def intranode(
        cls,
        max_num_tokens: int,
        num_experts: int,
        experts_per_token: int,
        rank: int,
        world_size: int,
        dp_size: int,
        hidden_dim: int,
        hidden_dim_bytes: int,
        hidden_dim_scale_bytes: int,
        group_name: str = "default",
    ) -> "AllToAll":
        assert world_size % dp_size == 0
        has_scales = hidden_dim_scale_bytes > 0
        if world_size > 1:
            group_name = _resolve_group_name(group_name)
        ptr = _ops.all_to_all_intranode_create(
            max_num_tokens,
            num_experts,
            experts_per_token,
            rank,
            world_size,
            dp_size,
            hidden_dim,
            hidden_dim_bytes,
            hidden_dim_scale_bytes,
            group_name,
        )
        assert ptr != 0
        return cls(
            ptr,
            _ops.all_to_all_intranode_combine,
            _ops.all_to_all_intranode_dispatch,
            has_scales,
        )

    @classmethod
    def internode(
        cls,
        max_num_tokens: int,
        num_experts: int,
        experts_per_token: int,
        rank: int,
        world_size: int,
        dp_size: int,
        hidden_dim: int,
        hidden_dim_bytes: int,
        hidden_dim_scale_bytes: int,
    ) -> "AllToAll":
        assert world_size % dp_size == 0
        has_scales = hidden_dim_scale_bytes > 0
        ptr = _ops.all_to_all_internode_create(
            max_num_tokens,
            num_experts,
            experts_per_token,
            rank,
            world_size,
            dp_size,
            hidden_dim,
            hidden_dim_bytes,
            hidden_dim_scale_bytes,
        )
        assert ptr != 0
        return cls(
            ptr,
            _ops.all_to_all_internode_combine,
            _ops.all_to_all_internode_dispatch,
            has_scales,
        )

    @classmethod
    def local_world(
        cls,
        max_num_tokens: int,
        num_experts: int,
        experts_per_token: int,
        world_size: int,
        dp_size: int,
        hidden_dim: int,
        hidden_dim_bytes: int,
        hidden_dim_scale_bytes: int,
    ) -> list["AllToAll"]:
        """``world_size`` ranks that all live on the current GPU of this process.

        They must be driven together with ``dispatch_group`` / ``combine_group``:
        ranks wait on one another, so they have to run inside one launch.
        """
        assert world_size % dp_size == 0
        ptrs = _ops.all_to_all_local_world_create(
            max_num_tokens,
            num_experts,
            experts_per_token,
            world_size,
            dp_size,
            hidden_dim,
            hidden_dim_bytes,
            hidden_dim_scale_bytes,
        )
        has_scales = hidden_dim_scale_bytes > 0
        return [
            cls(p, _ops.all_to_all_intranode_combine, _ops.all_to_all_intranode_dispatch, has_scales)
            for p in ptrs
        ]


def _or_empty(t: torch.Tensor | None, device: torch.device) -> torch.Tensor:
    return t if t is not None else torch.empty(0, device=device)


def dispatch_group(
    ranks: Sequence[AllToAll],
    out_expert_num_tokens: Sequence[torch.Tensor],
    out_expert_x: Sequence[torch.Tensor],
    out_expert_x_scale: Sequence[torch.Tensor | None],
    dp_x: Sequence[torch.Tensor],
    dp_x_scale: Sequence[torch.Tensor | None],
    indices: Sequence[torch.Tensor],
    bound_m: Sequence[torch.Tensor | None],
    do_send: bool = True,
    do_recv: bool = True,
) -> None:
    """One dispatch of every rank of a local world, as a single cooperative launch."""
    dev = dp_x[0].device
    _ops.all_to_all_dispatch_group(
        [r._ptr for r in ranks],
        list(out_expert_num_tokens),
        list(out_expert_x),
        [_or_empty(t, dev) for t in out_expert_x_scale],
        list(dp_x),
        [_or_empty(t, dev) for t in dp_x_scale],
        list(indices),
        [_or_empty(t, dev) for t in bound_m],
        do_send,
        do_recv,
    )


def combine_group(
    ranks: Sequence[AllToAll],
    out_tokens: Sequence[torch.Tensor],
    indices: Sequence[torch.Tensor],
    weights: Sequence[torch.Tensor],
    expert_y: Sequence[torch.Tensor],
    bound_m: Sequence[torch.Tensor | None],
    do_send: bool = True,
    do_recv: bool = True,
) -> None:
    """One combine of every rank of a local world, as a single cooperative launch."""
    dev = expert_y[0].device
    _ops.all_to_all_combine_group(
        [r._ptr for r in ranks],
        list(out_tokens),
        list(indices),
        list(weights),
        list(expert_y),
        [_or_empty(t, dev) for t in bound_m],
        do_send,
        do_recv,
    )


def fused_dispatch_group(
    ranks: Sequence[AllToAll],
    dp_x: Sequence[torch.Tensor],
    indices: Sequence[torch.Tensor],
    bound_m: Sequence[torch.Tensor | None],
    quantize: bool = False,
) -> None:
    """``fused_dispatch`` of every rank of a local world, as a single cooperative launch."""
    dev = dp_x[0].device
    _ops.moe_dispatch_send_group(
        [r._ptr for r in ranks], list(dp_x), list(indices), [_or_empty(t, dev) for t in bound_m],
        quantize,
    )
