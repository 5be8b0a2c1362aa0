"""Shared helpers for tests and benchmarks: MoE shapes, synthetic routing data
and a process launcher.

Role parity: tests/all_to_all_utils.py:6-56 (MoEConfig, RankTestData) and
tests/distributed_utils.py:17-136 (parallel_launch, ProcessGroupInfo) of the
reference, which keeps them next to its tests; they live in the package here
because bench.py and the examples use them too.
"""

from __future__ import annotations

import dataclasses
import os
import socket
from collections.abc import Callable
from typing import Any

import torch

from ..ops.reference import RankInputs


@dataclasses.dataclass
class MoEConfig:
    num_experts: int
    experts_per_token: int
    hidden_dim: int
    max_num_tokens: int
    in_dtype: torch.dtype = torch.bfloat16
    out_dtype: torch.dtype = torch.bfloat16
    block_size: int = 128

    @property
    def hidden_dim_bytes(self) -> int:
        return self.hidden_dim * self.in_dtype.itemsize

    @property
    def hidden_dim_scale(self) -> int:
        """Number of fp32 scales per token (0 unless the payload is 8-bit)."""
        if self.in_dtype.itemsize != 1:
            return 0
        return (self.hidden_dim + self.block_size - 1) // self.block_size

    @property
    def hidden_dim_scale_bytes(self) -> int:
        return self.hidden_dim_scale * 4


# Named shapes used by the tests, the benchmark and the documentation.
SMALL_MOE = MoEConfig(num_experts=8, experts_per_token=3, hidden_dim=512, max_num_tokens=10)
MEDIUM_MOE = MoEConfig(num_experts=64, experts_per_token=4, hidden_dim=1024, max_num_tokens=20)
DEEPSEEK_V3 = MoEConfig(num_experts=256, experts_per_token=8, hidden_dim=7168, max_num_tokens=128,
                        in_dtype=torch.float8_e4m3fn)
DEEPSEEK_V2_LITE = MoEConfig(num_experts=64, experts_per_token=6, hidden_dim=2048,
                             max_num_tokens=128, in_dtype=torch.float8_e4m3fn)


def routing(num_tokens: int, num_experts: int, topk: int, gen: torch.Generator,
            zipf: float = 0.0) -> torch.Tensor:
    """[num_tokens, topk] distinct experts per token, uniform or Zipf(zipf)-skewed."""
    if zipf > 0.0:
        p = 1.0 / torch.arange(1, num_experts + 1, dtype=torch.float64) ** zipf
    else:
        p = torch.ones(num_experts, dtype=torch.float64)
    p = (p / p.sum()).expand(max(num_tokens, 1), num_experts)
    idx = torch.multinomial(p, topk, replacement=False, generator=gen)
    return idx[:num_tokens].to(torch.int32)


def make_rank_inputs(cfg: MoEConfig, gen: torch.Generator, num_tokens: int | None = None,
                     zipf: float = 0.0, softmax_weights: bool = False) -> RankInputs:
    """Random tokens, routing and weights of one DP group (CPU tensors)."""
    if num_tokens is None:
        num_tokens = int(torch.randint(1, cfg.max_num_tokens + 1, [1], generator=gen).item())
    m = num_tokens
    indices = routing(m, cfg.num_experts, cfg.experts_per_token, gen, zipf)
    if softmax_weights:
        weights = torch.softmax(torch.randn(m, cfg.experts_per_token, generator=gen), dim=-1)
    else:
        weights = torch.rand(m, cfg.experts_per_token, generator=gen)
    x_scale = None
    if cfg.in_dtype.itemsize == 1:
        x = ((torch.rand(m, cfg.hidden_dim, generator=gen) - 0.5) * 400).to(cfg.in_dtype)
        x_scale = torch.rand(m, cfg.hidden_dim_scale, generator=gen)
    else:
        x = torch.randn(m, cfg.hidden_dim, generator=gen).to(cfg.in_dtype)
    return RankInputs(x=x, x_scale=x_scale, indices=indices, weights=weights.float(), num_tokens=m)


def as_index_tensor(indices: torch.Tensor, device: torch.device | str) -> torch.Tensor:
    """Routing indices in the dtype the kernels expect (uint32), on `device`."""
    return indices.to(torch.int32).to(device).view(torch.uint32)


# ------------------------------------------------------------------ launcher ----


@dataclasses.dataclass
class ProcessGroupInfo:
    world_size: int
    world_local_size: int
    rank: int
    node_rank: int
    local_rank: int
    device: torch.device


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(local_rank: int, world_size: int, port: int, use_cuda: bool,
            worker: Callable[..., None], args: tuple[Any, ...]) -> None:
    import torch.distributed as dist

    if use_cuda:
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        backend = "cpu:gloo,cuda:nccl"
    else:
        device = torch.device("cpu")
        backend = "gloo"
    dist.init_process_group(
        backend=backend,
        init_method=f"tcp://127.0.0.1:{port}",
        world_size=world_size,
        rank=local_rank,
    )
    try:
        pgi = ProcessGroupInfo(world_size, world_size, local_rank, 0, local_rank, device)
        worker(pgi, *args)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def parallel_launch(world_size: int, worker: Callable[..., None], *args: Any,
                    use_cuda: bool | None = None) -> None:
    """Runs ``worker(pgi, *args)`` in ``world_size`` spawned processes on this host.

    With CUDA each process owns the GPU of its rank and the default group is
    gloo (CPU tensors) + NCCL (CUDA tensors); without, gloo only.
    """
    if use_cuda is None:
        use_cuda = torch.cuda.is_available()
    os.environ.setdefault("NCCL_NVLS_ENABLE", os.environ.get("NCCL_NVLS_ENABLE", "0"))
    torch.multiprocessing.spawn(
        _worker,
        args=(world_size, free_port(), use_cuda, worker, args),
        nprocs=world_size,
        join=True,
    )


def _worker_from_env(local_rank: int, world_size: int, local_size: int, node_rank: int,
                     addr: str, port: int, use_cuda: bool, worker: Callable[..., None],
                     args: tuple[Any, ...]) -> None:
    import torch.distributed as dist

    rank = node_rank * local_size + local_rank
    if use_cuda:
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        backend = "cpu:gloo,cuda:nccl"
    else:
        device = torch.device("cpu")
        backend = "gloo"
    dist.init_process_group(backend=backend, init_method=f"tcp://{addr}:{port}",
                            world_size=world_size, rank=rank)
    try:
        pgi = ProcessGroupInfo(world_size, local_size, rank, node_rank, local_rank, device)
        worker(pgi, *args)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def launch_env_present() -> bool:
    """True when the variables `parallel_launch_from_env` reads are all set."""
    return all(k in os.environ for k in ("WORLD_SIZE", "WORLD_LOCAL_SIZE", "NODE_RANK",
                                         "MASTER_ADDR", "MASTER_PORT"))


def parallel_launch_from_env(worker: Callable[..., None], *args: Any,
                             use_cuda: bool | None = None) -> None:
    """Runs ``worker(pgi, *args)`` in ``WORLD_LOCAL_SIZE`` processes of this host as ranks
    ``NODE_RANK * WORLD_LOCAL_SIZE + local rank`` of a ``WORLD_SIZE`` job that meets at
    ``MASTER_ADDR:MASTER_PORT``.

    Role parity: ``parallel_launch_from_env`` of the reference (tests/distributed_utils.py:
    119-136), which starts its multi-node tests this way.  An `AllToAll` object of this
    library spans one NVLink domain, so `WORLD_SIZE` normally equals `WORLD_LOCAL_SIZE`; the
    launcher itself does not care.
    """
    world_size = int(os.environ["WORLD_SIZE"])
    local_size = int(os.environ["WORLD_LOCAL_SIZE"])
    node_rank = int(os.environ["NODE_RANK"])
    addr = os.environ["MASTER_ADDR"]
    port = int(os.environ["MASTER_PORT"])
    assert world_size % local_size == 0 and 0 <= node_rank < world_size // local_size
    if use_cuda is None:
        use_cuda = torch.cuda.is_available()
    os.environ.setdefault("NCCL_NVLS_ENABLE", os.environ.get("NCCL_NVLS_ENABLE", "0"))
    torch.multiprocessing.spawn(
        _worker_from_env,
        args=(world_size, local_size, node_rank, addr, port, use_cuda, worker, args),
        nprocs=local_size,
        join=True,
    )
