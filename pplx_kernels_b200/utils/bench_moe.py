"""Tokens/s of the MoE layer (dispatch -> expert FFN -> combine), fused vs composed.

    python -m pplx_kernels_b200.utils.bench_moe --model mixtral-8x7b --tokens 512
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m pplx_kernels_b200.utils.bench_moe --model mixtral-8x7b --tokens 512

One process per GPU (EP = world size).  CUDA-event timing per forward pass, L2
flushed between passes, maximum over ranks, p50 over iterations.  Rank 0 prints
one JSON line with both variants and the roofline of the layer: the slower of
expert FLOPs at the measured bf16 peak, expert weights over measured HBM
bandwidth, and activations over NVLink.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from pplx_kernels_b200.models.configs import CONFIGS
from pplx_kernels_b200.models.moe import MoELayer, MoELayerFP8
from pplx_kernels_b200.utils.testing import as_index_tensor, routing


def measure(model: str, tokens: int, iters: int, warmup: int, rank: int, world: int,
            dev: torch.device, zipf: float = 0.0, graph: bool = False,
            flush: torch.Tensor | None = None) -> dict:
    """Times the MoE layer of `model` at `tokens` per GPU, composed and fused.  With more than one
    rank torch.distributed must be initialised (NCCL for CUDA tensors)."""
    cfg = CONFIGS[model]
    m = tokens
    layer = MoELayer(cfg, max_num_tokens=m, rank=rank, world_size=world, device=dev)
    if world > 1:
        torch.distributed.barrier()  # weight initialisation takes a different time per rank
    gen = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(m, cfg.hidden_dim, generator=gen).to(torch.bfloat16).to(dev)
    idx = as_index_tensor(routing(m, cfg.num_experts, cfg.experts_per_token, gen, zipf), dev)
    w = torch.softmax(torch.randn(m, cfg.experts_per_token, generator=gen), dim=-1).to(dev)
    out = torch.zeros(m, cfg.hidden_dim, dtype=torch.bfloat16, device=dev)
    if flush is None:
        flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)

    def barrier() -> None:
        if world > 1:
            torch.distributed.barrier()

    res = {}
    for name, fused in (("composed", False), ("fused", True)):
        cuda_graph = None
        if graph:
            layer(x, idx, w, out=out, fused=fused)
            torch.cuda.synchronize()
            barrier()
            stream = torch.cuda.Stream()
            cuda_graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream), torch.cuda.graph(cuda_graph, stream=stream):
                layer(x, idx, w, out=out, fused=fused)
        times = []
        for it in range(warmup + iters):
            flush.add_(1)
            torch.cuda.synchronize()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if cuda_graph is not None:
                cuda_graph.replay()
            else:
                layer(x, idx, w, out=out, fused=fused)
            e1.record()
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(e0.elapsed_time(e1) * 1e3)
        t = torch.tensor(times, dtype=torch.float64, device=dev)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        res[name] = float(t.median())
    layer.check_status()
    layer.destroy()

    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    try:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    # Per GPU: rows = tokens * top-k (uniform routing, weak scaling)
    rows = m * cfg.experts_per_token
    flops = rows * 6 * cfg.hidden_dim * cfg.intermediate_dim
    nle = cfg.num_experts // world
    weight_bytes = nle * 3 * cfg.hidden_dim * cfg.intermediate_dim * 2
    wire_bytes = rows * cfg.hidden_dim * 2 * (world - 1) / world  # each way
    floors = {
        "compute_us": flops / (peaks["bf16_tflops"] * 1e6),
        "weights_hbm_us": weight_bytes / (peaks["hbm_gbs"] * 1e3),
        "nvlink_us_each_way": wire_bytes / 770e3,
    }
    floor = max(floors["compute_us"], floors["weights_hbm_us"], 2 * floors["nvlink_us_each_way"])
    best = min(res["fused"], res["composed"])
    return {
        "model": cfg.name, "n_gpus": world, "tokens_per_gpu": m, "graph": graph, "zipf": zipf,
        "composed_us_p50": res["composed"], "fused_us_p50": res["fused"],
        "fused_tokens_per_s": world * m / (res["fused"] * 1e-6),
        "composed_tokens_per_s": world * m / (res["composed"] * 1e-6),
        "floors_us": floors,
        "fused_frac_of_roofline": floor / res["fused"],
        "best_frac_of_roofline": floor / best,
    }


def measure_fp8(model: str, tokens: int, iters: int, warmup: int, rank: int, world: int,
                dev: torch.device, graph: bool = True, replays: int = 1) -> dict:
    """The fp8 layer (quantising dispatch -> fp8 GEMMs -> combine); with `graph` the forward
    pass is captured once and each timed sample is `replays` back-to-back replays."""
    cfg = CONFIGS[model]
    m = tokens
    layer = MoELayerFP8(cfg, max_num_tokens=m, rank=rank, world_size=world, device=dev)
    gen = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(m, cfg.hidden_dim, generator=gen).to(torch.bfloat16).to(dev)
    idx = as_index_tensor(routing(m, cfg.num_experts, cfg.experts_per_token, gen), dev)
    w = torch.softmax(torch.randn(m, cfg.experts_per_token, generator=gen), dim=-1).to(dev)
    out = torch.zeros(m, cfg.hidden_dim, dtype=torch.bfloat16, device=dev)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    layer(x, idx, w, out=out)
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    cuda_graph = None
    if graph:
        stream = torch.cuda.Stream()
        cuda_graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream), torch.cuda.graph(cuda_graph, stream=stream):
            layer(x, idx, w, out=out)
    times = []
    for it in range(warmup + iters):
        flush.add_(1)
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            if cuda_graph is not None:
                cuda_graph.replay()
            else:
                layer(x, idx, w, out=out)
        e1.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(e0.elapsed_time(e1) * 1e3 / replays)
    t = torch.tensor(times, dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    layer.check_status()
    layer.destroy()
    nle = cfg.num_experts // world
    weight_bytes = nle * 3 * cfg.hidden_dim * cfg.intermediate_dim  # one byte per weight
    us = float(t.median())
    return {"model": cfg.name, "dtype": "fp8 block-scaled", "n_gpus": world, "tokens_per_gpu": m,
            "graph": graph, "replays_per_sample": replays, "us_per_layer_p50": us,
            "tokens_per_s": world * m / (us * 1e-6),
            "weights_hbm_floor_us": weight_bytes / 6542e3}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=sorted(CONFIGS), default="mixtral-8x7b")
    ap.add_argument("--tokens", type=int, default=512, help="tokens per GPU")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--zipf", type=float, default=0.0)
    ap.add_argument("--graph", action="store_true", help="time CUDA-graph replays")
    ap.add_argument("--fp8", action="store_true", help="block-scaled fp8 layer (MoELayerFP8)")
    ap.add_argument("--replays", type=int, default=1, help="graph replays per timed sample")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        torch.distributed.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=dev)
    if args.fp8:
        row = measure_fp8(args.model, args.tokens, args.iters, args.warmup, rank, world, dev,
                          args.graph, args.replays)
    else:
        row = measure(args.model, args.tokens, args.iters, args.warmup, rank, world, dev,
                      args.zipf, args.graph)
    if rank == 0:
        print(json.dumps(row))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
