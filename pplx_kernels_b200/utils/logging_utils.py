"""Per-rank logging for multi-process runs.

Role parity: tests/logging_utils.py:4-10 of the reference (a root-logger format that carries the
process name) and the DEBUG dumps of routing in its test (tests/test_all_to_all.py:123-150).
"""

from __future__ import annotations

import logging
import os

import torch


def init_logging(rank: int | None = None, level: int | str | None = None) -> logging.Logger:
    """Configures the root logger with a ``[rank r]`` prefix and returns the package logger.

    `rank` defaults to the ``RANK`` environment variable; `level` to ``PPLX_B200_LOG_LEVEL``
    (a name such as ``DEBUG``), else INFO.  Calling it again replaces the format.
    """
    if rank is None:
        rank = int(os.environ.get("RANK", "0"))
    if level is None:
        level = os.environ.get("PPLX_B200_LOG_LEVEL", "INFO")
    logging.basicConfig(
        level=level,
        format=f"%(asctime)s [rank {rank}] %(levelname)s %(name)s: %(message)s",
        force=True,
    )
    return logging.getLogger("pplx_kernels_b200")


def describe_routing(indices: torch.Tensor, num_experts: int, world_size: int) -> str:
    """One line per destination rank: how many (token, k) entries of `indices` go there and
    the per-expert histogram, for DEBUG logs of a test or a serving step."""
    idx = indices.detach().to("cpu").to(torch.int64).flatten()
    idx = idx[(idx >= 0) & (idx < num_experts)]
    hist = torch.bincount(idx, minlength=num_experts)
    nle = -(-num_experts // world_size)
    lines = []
    for r in range(world_size):
        part = hist[r * nle:min((r + 1) * nle, num_experts)]
        lines.append(f"rank {r}: {int(part.sum())} rows, per expert {part.tolist()}")
    return "\n".join(lines)
