"""Profiling driver for the dispatch and combine kernels.

    python -m pplx_kernels_b200.utils.profile_a2a --tokens 128 --iters 20 --trace
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m pplx_kernels_b200.utils.profile_a2a --tokens 128 --iters 20 --trace

runs the DeepSeek-V3 shape (256 experts, top-8, hidden 7168, fp8 + scales in,
bf16 out), prints CUDA-event latencies and, with ``--trace``, the per-phase
breakdown that block 0 stamps with %globaltimer (rank 0's, when started with one
process per GPU).  With one rank and few iterations it is also the command to put
under ``ncu`` (one kernel, a few launches).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

import pplx_kernels_b200 as pk
from pplx_kernels_b200.utils.testing import MoEConfig, as_index_tensor, make_rank_inputs


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--max-blocks", type=int, default=0)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=dev)
        uid = pk.nvshmem_get_unique_id() if rank == 0 else pk.nvshmem_alloc_empty_unique_id()
        dist.broadcast(uid, src=0)
        pk.nvshmem_init(uid, rank, world)

    def rank_barrier() -> None:
        if world > 1:
            pk.nvshmem_barrier_all_on_current_stream()

    cfg = MoEConfig(args.experts, args.topk, args.hidden, args.tokens,
                    in_dtype=torch.float8_e4m3fn, out_dtype=torch.bfloat16)
    inp = make_rank_inputs(cfg, torch.Generator().manual_seed(1 + rank), num_tokens=args.tokens,
                           softmax_weights=True)
    ata = pk.AllToAll.intranode(cfg.max_num_tokens, cfg.num_experts, cfg.experts_per_token, rank,
                                world, 1, cfg.hidden_dim, cfg.hidden_dim_bytes,
                                cfg.hidden_dim_scale_bytes)
    if args.max_blocks:
        ata.set_max_blocks(args.max_blocks)
    ata.set_trace(args.trace)
    x, xs = inp.x.to(dev), inp.x_scale.to(dev)
    idx, w = as_index_tensor(inp.indices, dev), inp.weights.to(dev)
    bound_m = torch.tensor([args.tokens], dtype=torch.int32, device=dev).view(torch.uint32)
    nle, rows = cfg.num_experts // world, args.tokens * world
    counts = torch.zeros(nle, dtype=torch.int32, device=dev)
    ex = torch.zeros(nle, rows, cfg.hidden_dim, dtype=torch.uint8, device=dev).view(cfg.in_dtype)
    es = torch.zeros(nle, rows, cfg.hidden_dim_scale, device=dev)
    ey = torch.randn(nle, rows, cfg.hidden_dim, device=dev).to(cfg.out_dtype)
    out = torch.zeros(args.tokens, cfg.hidden_dim, dtype=cfg.out_dtype, device=dev)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)

    from pplx_kernels_b200.ops import _ops

    lat = {"dispatch": [], "combine": [], "empty_kernel": []}
    phases: dict[str, list[float]] = {}
    for it in range(args.warmup + args.iters):
        if not args.no_flush:
            flush.add_(1)
        rank_barrier()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        ata.dispatch(counts, ex, es, x, xs, idx, bound_m)
        e[1].record()
        ata.combine(out, idx, w, ey, bound_m)
        e[2].record()
        torch.cuda.synchronize()
        # Calibration: the same event bracket around a kernel that does nothing.
        if not args.no_flush:
            flush.add_(1)
        c = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        c[0].record()
        _ops.sleep_on_stream(0.0)
        c[1].record()
        torch.cuda.synchronize()
        if it < args.warmup:
            continue
        lat["empty_kernel"].append(c[0].elapsed_time(c[1]) * 1e3)
        lat["dispatch"].append(e[0].elapsed_time(e[1]) * 1e3)
        lat["combine"].append(e[1].elapsed_time(e[2]) * 1e3)
        if args.trace:
            t = ata.read_trace()
            order = ["dispatch_start", "dispatch_hist", "dispatch_posted", "dispatch_stored",
                     "dispatch_signalled", "dispatch_counts", "dispatch_layout",
                     "dispatch_copied", "dispatch_end"]
            for a, b in zip(order, order[1:], strict=False):
                phases.setdefault(f"{a}->{b}", []).append((t[b] - t[a]) / 1e3)
            order = ["combine_start", "combine_layout", "combine_sent", "combine_reduced",
                     "combine_end"]
            for a, b in zip(order, order[1:], strict=False):
                phases.setdefault(f"{a}->{b}", []).append((t[b] - t[a]) / 1e3)
            for op in ("dispatch", "combine"):
                k = op + "_blocks"
                phases.setdefault(f"{op}: first block start -> last block start", []).append(
                    (t[k + "_last_start"] - t[k + "_first_start"]) / 1e3)
                phases.setdefault(f"{op}: first block start -> first block end", []).append(
                    (t[k + "_first_end"] - t[k + "_first_start"]) / 1e3)
                phases.setdefault(f"{op}: first block start -> last block end", []).append(
                    (t[k + "_last_end"] - t[k + "_first_start"]) / 1e3)
            phases.setdefault("dispatch last end -> combine first start", []).append(
                (t["combine_blocks_first_start"] - t["dispatch_blocks_last_end"]) / 1e3)
    ata.check_status()
    ata.destroy()
    report = {
        "tokens": args.tokens,
        "world": world,
        "dispatch_us_p50": statistics.median(lat["dispatch"]),
        "combine_us_p50": statistics.median(lat["combine"]),
        "empty_kernel_us_p50": statistics.median(lat["empty_kernel"]),
        "phases_us_p50": {k: statistics.median(v) for k, v in phases.items()},
    }
    if rank == 0:
        print(json.dumps(report, indent=1))
    if world > 1:
        torch.distributed.barrier()
        pk.nvshmem_finalize()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
