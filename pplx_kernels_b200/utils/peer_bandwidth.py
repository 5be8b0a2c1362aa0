"""Peer-store bandwidth of this machine, as a plain copy kernel of the library sees it.

Every rank stores one chunk into every rank's symmetric buffer at the same time (the dense
all-to-all kernel behind ``nvshmem_alltoall``: 16-byte stores from registers, followed by the
stream barrier).  The bytes a rank pushes through its NVLink ports divided by the CUDA-event
time, minimum over ranks, is the ceiling that the dispatch and combine kernels are compared
with: they move their payload with the same kind of store.
"""

from __future__ import annotations

import torch

from ..nvshmem import nvshmem_alltoall, nvshmem_malloc, nvshmem_n_pes


def measure_peer_store_gbs(chunk_mib: int = 64, iters: int = 5) -> float:
    """GB/s per direction and GPU; needs the symmetric-memory runtime (``nvshmem_init``) and
    torch.distributed for the minimum over ranks."""
    world = nvshmem_n_pes()
    if world < 2:
        raise RuntimeError("peer bandwidth needs at least two ranks")
    dev = torch.device("cuda", torch.cuda.current_device())
    chunk = chunk_mib << 20
    dst = nvshmem_malloc([world, chunk], torch.uint8, dev)
    src = torch.zeros(world, chunk, dtype=torch.uint8, device=dev)
    best = 0.0
    for it in range(iters + 2):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.distributed.barrier()
        e0.record()
        nvshmem_alltoall(dst, src)
        e1.record()
        torch.cuda.synchronize()
        if it >= 2:
            best = max(best, (world - 1) * chunk / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    t = torch.tensor([best], device=dev)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
    del dst
    return float(t.item())
