"""Blackwell-native MoE expert-parallel all-to-all (dispatch / combine).

The public names mirror ``pplx_kernels`` (src/pplx_kernels/__init__.py:1-16 of
the reference) so that existing callers can switch the import.
"""

from . import ops as ops
from .all_to_all import (
    AllToAll as AllToAll,
    combine_group as combine_group,
    dispatch_group as dispatch_group,
    fused_dispatch_group as fused_dispatch_group,
)
from .nvshmem import (
    nvshmem_alloc_empty_unique_id as nvshmem_alloc_empty_unique_id,
    nvshmem_alltoall as nvshmem_alltoall,
    nvshmem_barrier_all as nvshmem_barrier_all,
    nvshmem_barrier_all_on_current_stream as nvshmem_barrier_all_on_current_stream,
    nvshmem_finalize as nvshmem_finalize,
    nvshmem_get_unique_id as nvshmem_get_unique_id,
    nvshmem_init as nvshmem_init,
    nvshmem_malloc as nvshmem_malloc,
    nvshmem_my_pe as nvshmem_my_pe,
    nvshmem_n_pes as nvshmem_n_pes,
    nvshmem_unique_id_size as nvshmem_unique_id_size,
)

__version__ = "0.1.0"
