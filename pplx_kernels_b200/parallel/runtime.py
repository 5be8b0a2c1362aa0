"""Bring up the process-wide symmetric-memory runtime from an initialised
``torch.distributed`` job: rank 0 creates the rendezvous id, everybody receives it
through a broadcast (what the reference's tests do with the NVSHMEM unique id,
tests/test_all_to_all.py:296-300)."""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..nvshmem import (
    nvshmem_alloc_empty_unique_id,
    nvshmem_finalize,
    nvshmem_get_unique_id,
    nvshmem_init,
)


def init_runtime_from_torch(group: dist.ProcessGroup | None = None) -> tuple[int, int]:
    """Returns (rank, world_size) after ``nvshmem_init``.  Works without torch.distributed
    (single process) as well."""
    if not dist.is_available() or not dist.is_initialized():
        nvshmem_init(nvshmem_get_unique_id(), 0, 1)
        return 0, 1
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    uid = nvshmem_get_unique_id() if rank == 0 else nvshmem_alloc_empty_unique_id()
    src = dist.get_global_rank(group, 0) if group is not None else 0
    dist.broadcast(uid, src=src, group=group)
    nvshmem_init(uid, rank, world)
    return rank, world


def finalize_runtime() -> None:
    if torch.cuda.is_available():
        nvshmem_finalize()
