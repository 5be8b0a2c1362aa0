"""Sweep benchmark of dispatch / combine against generic all-to-all baselines.

    python -m pplx_kernels_b200.utils.bench_all_to_all                    # one GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m pplx_kernels_b200.utils.bench_all_to_all --tokens 1,128,1024,4096 --zipf 1.2

Role parity: tests/bench_all_to_all.py:32-368 of the reference -- the same two
model shapes (DeepSeek-V2-Lite 64 experts / top-6 / hidden 2048 and R1 256 /
top-8 / 7168), the same four timed operations per sample (dispatch, combine,
torch ``all_to_all_single`` and the symmetric-memory all-to-all on the dense
``[world, local experts, tokens * bytes]`` shape) and a TSV in ``data/``.
Differences: one process per GPU is started by torchrun, every number is the
maximum over ranks of CUDA-event times, p50 is reported next to mean +- std,
token counts up to 4096 and Zipf-skewed routing are supported, and each row
carries the NVLink (or, on one GPU, HBM) floor of the operation.
"""

from __future__ import annotations

import argparse
import json
import os
import time
from pathlib import Path

import torch

import pplx_kernels_b200 as pk
from pplx_kernels_b200.utils.testing import MoEConfig, as_index_tensor, make_rank_inputs

NVLINK_GBS = 770.0


def _max_over_ranks(t: torch.Tensor, world: int) -> torch.Tensor:
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return t


def bench_config(cfg: MoEConfig, rank: int, world: int, dev: torch.device, zipf: float,
                 repeat: int, samples: int, warmup: int, flush: torch.Tensor | None,
                 dp_size: int = 1) -> dict:
    nle = cfg.num_experts // world
    # The ranks of one DP group hold the same tokens.
    gen = torch.Generator().manual_seed(7 + rank // dp_size)
    inp = make_rank_inputs(cfg, gen, num_tokens=cfg.max_num_tokens, zipf=zipf)
    ata = pk.AllToAll.internode(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token, rank,
                                world, dp_size, cfg.hidden_dim, cfg.hidden_dim_bytes,
                                cfg.hidden_dim_scale_bytes)
    layout = ata.layout()
    rows = cfg.max_num_tokens * world
    counts = torch.empty(nle, dtype=torch.int32, device=dev)
    expert_x = torch.empty(nle, rows, cfg.hidden_dim, dtype=torch.uint8 if cfg.in_dtype.itemsize == 1
                           else cfg.in_dtype, device=dev)
    if cfg.in_dtype.itemsize == 1:
        expert_x = expert_x.view(cfg.in_dtype)
    expert_scale = None
    x_scale = None
    if cfg.hidden_dim_scale:
        expert_scale = torch.empty(nle, rows, cfg.hidden_dim_scale, device=dev)
        x_scale = inp.x_scale.to(dev)
    expert_y = torch.zeros(nle, rows, cfg.hidden_dim, dtype=cfg.out_dtype, device=dev)
    x = inp.x.to(dev)
    indices = as_index_tensor(inp.indices, dev)
    weights = inp.weights.to(dev)
    bound_m = torch.tensor([cfg.max_num_tokens], dtype=torch.int32, device=dev).view(torch.uint32)
    y = torch.empty(cfg.max_num_tokens, cfg.hidden_dim, dtype=cfg.out_dtype, device=dev)

    per_token = cfg.hidden_dim_bytes + cfg.hidden_dim_scale_bytes
    a2a_shape = (world, nle, cfg.max_num_tokens * per_token)
    a2a_bytes = world * nle * cfg.max_num_tokens * per_token
    dense_ok = a2a_bytes <= (2 << 30)
    if dense_ok:
        a2a_in = torch.zeros(a2a_shape, dtype=torch.uint8, device=dev)
        a2a_out = torch.empty_like(a2a_in)
        sym_in = pk.nvshmem_malloc(a2a_shape, torch.uint8, dev)
        sym_out = pk.nvshmem_malloc(a2a_shape, torch.uint8, dev)

    names = ["dispatch", "combine", "torch_all_to_all", "symm_all_to_all"]
    all_times: list[list[float]] = [[] for _ in names]
    stream = torch.cuda.current_stream()
    for rep in range(warmup + repeat):
        events = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(samples)]
        for e in events:
            if flush is not None:
                flush.add_(1)
            pk.nvshmem_barrier_all_on_current_stream()
            e[0].record(stream)
            ata.dispatch(counts, expert_x, expert_scale, x, x_scale, indices, bound_m)
            e[1].record(stream)
            ata.combine(y, indices, weights, expert_y, bound_m)
            e[2].record(stream)
            if dense_ok and world > 1:
                torch.distributed.all_to_all_single(a2a_out, a2a_in)
            e[3].record(stream)
            if dense_ok:
                pk.nvshmem_alltoall(sym_out, sym_in)
            e[4].record(stream)
        stream.synchronize()
        if rep < warmup:
            continue
        for e in events:
            for k in range(4):
                all_times[k].append(e[k].elapsed_time(e[k + 1]) * 1e3)
    ata.check_status()
    ata.destroy()
    t = _max_over_ranks(torch.tensor(all_times, dtype=torch.float64, device=dev), world).cpu()
    row = {
        "experts": cfg.num_experts, "topk": cfg.experts_per_token, "hidden": cfg.hidden_dim,
        "tokens": cfg.max_num_tokens, "zipf": zipf, "ep": world, "dp_size": dp_size,
        "multicast": layout["multicast"],
    }
    disp_bytes = cfg.max_num_tokens * cfg.experts_per_token * per_token
    comb_bytes = cfg.max_num_tokens * cfg.experts_per_token * cfg.hidden_dim * cfg.out_dtype.itemsize
    # One GPU: nothing crosses NVLink; the floor is then local traffic (staging write +
    # staging read + output write) over the measured copy bandwidth, expressed through the
    # same formula with an equivalent "remote share".
    remote = (world - 1) / world if world > 1 else 3.0 * NVLINK_GBS / 6542.0
    for k, name in enumerate(names):
        if (name == "torch_all_to_all" and (world == 1 or not dense_ok)) or (
                name == "symm_all_to_all" and not dense_ok):
            row[name + "_us_p50"] = None
            continue
        row[name + "_us_mean"] = float(t[k].mean())
        row[name + "_us_std"] = float(t[k].std())
        row[name + "_us_p50"] = float(t[k].median())
    row["dispatch_bytes"] = disp_bytes
    row["combine_bytes"] = comb_bytes
    row["dispatch_floor_us"] = disp_bytes * remote / NVLINK_GBS / 1e3
    row["combine_floor_us"] = comb_bytes * remote / NVLINK_GBS / 1e3
    row["dispatch_frac_of_floor"] = row["dispatch_floor_us"] / row["dispatch_us_p50"]
    row["combine_frac_of_floor"] = row["combine_floor_us"] / row["combine_us_p50"]
    if dense_ok:
        del sym_in, sym_out
    return row


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,4,8,16,32,64,128")
    ap.add_argument("--shapes", default="v2lite,r1", help="comma list of v2lite, r1")
    ap.add_argument("--in-dtype", choices=["bfloat16", "float16", "float8_e4m3fn"],
                    default="float8_e4m3fn")
    ap.add_argument("--out-dtype", choices=["bfloat16", "float16"], default="bfloat16")
    ap.add_argument("--zipf", type=float, default=0.0, help="0 = uniform routing")
    ap.add_argument("--repeat", type=int, default=10)
    ap.add_argument("--samples", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--dp-size", type=int, default=1,
                    help="ranks that hold the same tokens (0: all of them)")
    ap.add_argument("--multimem-ab", action="store_true",
                    help="run every row twice in this process: arena from CUDA IPC, then from "
                         "driver allocations bound to an NVLink multicast object")
    ap.add_argument("--out-dir", default="data")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        torch.distributed.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=dev)
    uid = pk.nvshmem_get_unique_id() if rank == 0 else pk.nvshmem_alloc_empty_unique_id()
    if world > 1:
        torch.distributed.broadcast(uid, src=0)
    pk.nvshmem_init(uid, rank, world)

    shapes = {"v2lite": (64, 6, 2048), "r1": (256, 8, 7168)}
    in_dtype, out_dtype = getattr(torch, args.in_dtype), getattr(torch, args.out_dtype)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev) if args.flush_l2 else None
    rows = []
    # The arena's kind is read from the environment when an object is created.
    modes = ("0", "1") if args.multimem_ab else (os.environ.get("PPLX_B200_MULTIMEM", "0"),)
    for mode in modes:
        os.environ["PPLX_B200_MULTIMEM"] = mode
        if args.multimem_ab:
            os.environ["PPLX_B200_MULTIMEM_COMBINE"] = "1"  # the comparison is about this path
        for name in args.shapes.split(","):
            experts, topk, hidden = shapes[name]
            if experts % world:
                continue
            for tok in (int(t) for t in args.tokens.split(",")):
                cfg = MoEConfig(experts, topk, hidden, tok, in_dtype, out_dtype)
                row = bench_config(cfg, rank, world, dev, args.zipf, args.repeat, args.samples,
                                   args.warmup, flush, args.dp_size or world)
                row["shape"] = name
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
    if rank == 0:
        out_dir = Path(args.out_dir)
        out_dir.mkdir(parents=True, exist_ok=True)
        path = out_dir / f"{time.strftime('%Y%m%d_%H%M%S')}_all_to_all_ep{world}.tsv"
        cols = list(rows[0].keys()) if rows else []
        with path.open("w") as f:
            f.write("\t".join(cols) + "\n")
            for r in rows:
                f.write("\t".join("" if r.get(c) is None else str(r.get(c)) for c in cols) + "\n")
        print("saved", path)
    pk.nvshmem_finalize()
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
