"""Tokens/s of the MoE layer (dispatch -> expert FFN -> combine), fused vs composed.

    python -m pplx_kernels_b200.utils.bench_moe --model mixtral-8x7b --tokens 512
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m pplx_kernels_b200.utils.bench_moe --model qwen3-30b-a3b --fp8 --tokens 1,16,64,256 \
        --graph --replays 1000

One process per GPU (EP = world size).  Before anything is timed the layer's output, fused and
composed, is compared with the plain-PyTorch statement of the layer over the whole model's
weights (gathered from all ranks), so that a timing is never a timing of unknown work.  Then:
CUDA-event timing per forward pass, L2 flushed between samples, maximum over ranks, p50 over
iterations.  Rank 0 prints one JSON line per token count with both variants and the roofline
of the layer: the slowest of expert FLOPs at the measured bf16 peak, expert weights over
measured HBM bandwidth, and activations over NVLink.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from pplx_kernels_b200.models.configs import CONFIGS
from pplx_kernels_b200.models.moe import (
    MoELayer,
    MoELayerFP8,
    moe_reference,
    moe_reference_fp8,
)
from pplx_kernels_b200.utils.testing import as_index_tensor, routing

NVLINK_GBS = 770.0
# Largest model (parameters over all ranks) whose weights are gathered for the check.
VERIFY_MAX_PARAMS = 3_000_000_000


def _peaks() -> dict:
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    try:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    return peaks


def _gather(t: torch.Tensor, world: int) -> torch.Tensor:
    if world == 1:
        return t
    parts = [torch.empty_like(t) for _ in range(world)]
    torch.distributed.all_gather(parts, t.contiguous())
    return torch.cat(parts)


# fp8 layers: power-of-two scales applied by the tensor cores (--pow2).
POW2_SCALES = False


def _fp8_layer(cfg, **kw):
    return MoELayerFP8(cfg, pow2_scales=POW2_SCALES, **kw)


def verify_layer(layer, fp8: bool, x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor,
                 world: int) -> str:
    """Runs the layer composed and fused and compares both with the reference.  Returns how it
    was checked; raises on a mismatch."""
    cfg = layer.cfg
    dev = x.device
    idx_dev = as_index_tensor(idx, dev)
    m = x.size(0)
    outs = {}
    for name, fused in (("composed", False), ("fused", True)):
        outs[name] = layer(x, idx_dev, w, fused=fused)[:m].float().clone()
        torch.cuda.synchronize()
        layer.check_status()
    params = cfg.num_experts * 3 * cfg.hidden_dim * cfg.intermediate_dim
    def close(got: torch.Tensor, want: torch.Tensor, rel: float, of_max: float, what: str) -> None:
        # Elementwise: a share of the value plus a share of the largest value (a rounding of
        # an intermediate moves a small output by an amount that scales with the row).
        err = (got - want).abs()
        bound = rel * want.abs() + of_max * want.abs().amax()
        assert (err <= bound).all(), (
            f"{what}: largest error {float(err.max()):.4g} where {float(bound[err.argmax()] if err.dim() == 1 else bound.flatten()[err.argmax()]):.4g} "
            f"is allowed (largest value {float(want.abs().amax()):.4g})")

    # The two paths do the same arithmetic; they may differ by roundings of the top-k sums only.
    close(outs["fused"], outs["composed"], 2e-2, 5e-3, "fused against composed")
    if params > VERIFY_MAX_PARAMS:
        return "fused against composed (the model is too large to gather for the reference)"
    if fp8:
        w13, w2 = layer.dequantized_weights()
        want = moe_reference_fp8(x, idx.to(dev), w, _gather(w13, world), _gather(w2, world),
                                 pow2=POW2_SCALES)
        for name, out in outs.items():
            close(out, want, 0.06, 0.04, f"{name} against the fp8 reference")
    else:
        want = moe_reference(x, idx.to(dev), w, _gather(layer.w13, world), _gather(layer.w2, world))
        for name, out in outs.items():
            close(out, want, 3e-2, 1e-2, f"{name} against the reference")
    return "fused and composed against the PyTorch reference over all experts, and against each other"


def measure(model: str, tokens: int, iters: int, warmup: int, rank: int, world: int,
            dev: torch.device, zipf: float = 0.0, graph: bool = False,
            flush: torch.Tensor | None = None, fp8: bool = False, replays: int = 1,
            verify: bool = True) -> dict:
    """Times the MoE layer of `model` at `tokens` per GPU, composed and fused.  With more than one
    rank torch.distributed must be initialised (NCCL for CUDA tensors).  With `graph` a forward
    pass is captured once and every timed sample is `replays` back-to-back replays."""
    cfg = CONFIGS[model]
    m = tokens
    make = _fp8_layer if fp8 else MoELayer
    layer = make(cfg, max_num_tokens=m, rank=rank, world_size=world, device=dev)
    if world > 1:
        torch.distributed.barrier()  # weight initialisation takes a different time per rank
    gen = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(m, cfg.hidden_dim, generator=gen).to(torch.bfloat16).to(dev)
    idx_host = routing(m, cfg.num_experts, cfg.experts_per_token, gen, zipf)
    idx = as_index_tensor(idx_host, dev)
    w = torch.softmax(torch.randn(m, cfg.experts_per_token, generator=gen), dim=-1).to(dev)
    out = torch.zeros(m, cfg.hidden_dim, dtype=torch.bfloat16, device=dev)
    if flush is None:
        flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    checked = verify_layer(layer, fp8, x, idx_host, w, world) if verify else "not checked"

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
            for _ in range(replays if cuda_graph is not None else 1):
                if cuda_graph is not None:
                    cuda_graph.replay()
                else:
                    layer(x, idx, w, out=out, fused=fused)
            e1.record()
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(e0.elapsed_time(e1) * 1e3 / (replays if cuda_graph is not None else 1))
        t = torch.tensor(times, dtype=torch.float64, device=dev)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        res[name] = float(t.median())
    layer.check_status()
    layer.destroy()

    peaks = _peaks()
    # Per GPU: rows = tokens * top-k (uniform routing, weak scaling)
    rows = m * cfg.experts_per_token
    flops = rows * 6 * cfg.hidden_dim * cfg.intermediate_dim
    nle = cfg.num_experts // world
    # Weights that must stream from HBM: every local expert at large batches, at most one
    # expert per row at small ones; one byte per weight in fp8, two in bf16.
    touched = min(nle, rows)
    weight_bytes = touched * 3 * cfg.hidden_dim * cfg.intermediate_dim * (1 if fp8 else 2)
    wire_bytes = rows * cfg.hidden_dim * (world - 1) / world  # bytes per element below
    # The measured bf16 peak for both dtypes: it is the one GEMM peak measured on the box (the
    # fp8 tensor pipe is nominally twice as fast, so an fp8 layer can exceed this "floor").
    floors = {
        "compute_us": flops / (peaks["bf16_tflops"] * 1e6),
        "weights_hbm_us": weight_bytes / (peaks["hbm_gbs"] * 1e3),
        "nvlink_dispatch_us": wire_bytes * (1 if fp8 else 2) / (NVLINK_GBS * 1e3),
        "nvlink_combine_us": wire_bytes * 2 / (NVLINK_GBS * 1e3),
    }
    floor = max(floors["compute_us"], floors["weights_hbm_us"],
                floors["nvlink_dispatch_us"] + floors["nvlink_combine_us"])
    best = min(res["fused"], res["composed"])
    return {
        "model": cfg.name,
        "dtype": ("fp8 block-scaled, power-of-two scales applied by the tensor cores"
                  if fp8 and POW2_SCALES else "fp8 block-scaled" if fp8 else "bf16"),
        "n_gpus": world,
        "tokens_per_gpu": m, "graph": graph, "replays_per_sample": replays if graph else 1,
        "zipf": zipf, "output_checked": checked,
        "composed_us_p50": res["composed"], "fused_us_p50": res["fused"],
        "fused_tokens_per_s": world * m / (res["fused"] * 1e-6),
        "composed_tokens_per_s": world * m / (res["composed"] * 1e-6),
        "floors_us": floors,
        "fused_frac_of_roofline": floor / res["fused"],
        "best_frac_of_roofline": floor / best,
    }


def breakdown(model: str, tokens: int, iters: int, warmup: int, rank: int, world: int,
              dev: torch.device, fp8: bool = False) -> dict:
    """p50 microseconds of each of the four kernels of the layer, composed and fused (CUDA events
    between the calls, L2 flushed before each pass, max over ranks).  The events add a few
    microseconds per kernel; the figures are for comparing the kernels, not for the totals."""
    from pplx_kernels_b200.ops.grouped_gemm import grouped_gemm, grouped_gemm_fp8

    cfg = CONFIGS[model]
    m = tokens
    layer = (_fp8_layer if fp8 else MoELayer)(cfg, max_num_tokens=m, rank=rank, world_size=world,
                                              device=dev)
    gen = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(m, cfg.hidden_dim, generator=gen).to(torch.bfloat16).to(dev)
    idx = as_index_tensor(routing(m, cfg.num_experts, cfg.experts_per_token, gen), dev)
    w = torch.softmax(torch.randn(m, cfg.experts_per_token, generator=gen), dim=-1).to(dev)
    out = torch.zeros(m, cfg.hidden_dim, dtype=torch.bfloat16, device=dev)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    a, L = layer.ata, layer
    expect = m * cfg.experts_per_token
    if fp8:
        steps = {
            "composed": [
                ("dispatch_quant", lambda: a.dispatch_quant(L.counts, L.expert_x, L.expert_scale, x, idx, None)),
                ("up", lambda: grouped_gemm_fp8(L.expert_x, L.expert_scale, L.w13_q, L.w13_s, L.counts,
                                                swiglu_quant=True, out=L.h, out_scale=L.h_scale,
                                                status=L.gemm_status, pow2_scales=POW2_SCALES)),
                ("down", lambda: grouped_gemm_fp8(L.h, L.h_scale, L.w2_q, L.w2_s, L.counts,
                                                  out=L.expert_y, status=L.gemm_status,
                                                  pow2_scales=POW2_SCALES)),
                ("combine", lambda: a.combine(out, idx, w, L.expert_y, None))],
            "fused": [
                ("fused_dispatch", lambda: a.fused_dispatch(x, idx, None, quantize=True)),
                ("fused_up", lambda: a.fused_up_fp8(L.w13_q, L.w13_s, L.h, L.h_scale, L.counts, L.gemm_status)),
                ("fused_down", lambda: a.fused_down_fp8(L.h, L.h_scale, L.w2_q, L.w2_s, L.gemm_status)),
                ("combine_recv", lambda: a.combine(out, idx, w, L.expert_y, None, do_send=False))]}
    else:
        steps = {
            "composed": [
                ("dispatch", lambda: a.dispatch(L.counts, L.expert_x, None, x, None, idx, None)),
                ("up", lambda: grouped_gemm(L.expert_x, L.w13, L.counts, out=L.h, swiglu=True,
                                            status=L.gemm_status, expected_rows=expect)),
                ("down", lambda: grouped_gemm(L.h, L.w2, L.counts, out=L.expert_y, swiglu=False,
                                              status=L.gemm_status, expected_rows=expect)),
                ("combine", lambda: a.combine(out, idx, w, L.expert_y, None))],
            "fused": [
                ("fused_dispatch", lambda: a.fused_dispatch(x, idx, None)),
                ("fused_up", lambda: a.fused_up(L.w13, L.h, L.counts, L.gemm_status, expect)),
                ("fused_down", lambda: a.fused_down(L.h, L.w2, L.gemm_status, expect)),
                ("combine_recv", lambda: a.combine(out, idx, w, L.expert_y, None, do_send=False))]}
    report: dict = {"model": cfg.name, "n_gpus": world, "tokens_per_gpu": m, "fp8": fp8,
                    "pow2_scales": bool(fp8 and POW2_SCALES)}
    for variant, calls in steps.items():
        samples = []
        for it in range(warmup + iters):
            flush.add_(1)
            torch.cuda.synchronize()
            if world > 1:
                torch.distributed.barrier()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(calls) + 1)]
            ev[0].record()
            for k, (_, fn) in enumerate(calls):
                fn()
                ev[k + 1].record()
            torch.cuda.synchronize()
            if it >= warmup:
                samples.append([ev[k].elapsed_time(ev[k + 1]) * 1e3 for k in range(len(calls))]
                               + [ev[0].elapsed_time(ev[-1]) * 1e3])
        t = torch.tensor(samples, dtype=torch.float64, device=dev)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        med = t.median(dim=0).values.tolist()
        report[variant] = {name: med[k] for k, (name, _) in enumerate(calls)}
        report[variant]["total"] = med[-1]
    layer.check_status()
    layer.destroy()
    return report


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=sorted(CONFIGS), default="mixtral-8x7b")
    ap.add_argument("--tokens", default="512", help="tokens per GPU, or a comma list")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--zipf", type=float, default=0.0)
    ap.add_argument("--graph", action="store_true", help="time CUDA-graph replays")
    ap.add_argument("--fp8", action="store_true", help="block-scaled fp8 layer (MoELayerFP8)")
    ap.add_argument("--pow2", action="store_true",
                    help="with --fp8: power-of-two scales, applied by the tensor cores")
    ap.add_argument("--replays", type=int, default=1, help="graph replays per timed sample")
    ap.add_argument("--no-verify", action="store_true", help="skip the output check")
    ap.add_argument("--breakdown", action="store_true",
                    help="time each of the layer's four kernels instead of the layer")
    args = ap.parse_args()
    global POW2_SCALES
    POW2_SCALES = bool(args.fp8 and args.pow2)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        torch.distributed.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=dev)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    for tokens in (int(t) for t in args.tokens.split(",")):
        if args.breakdown:
            row = breakdown(args.model, tokens, args.iters, args.warmup, rank, world, dev, args.fp8)
            if rank == 0:
                print(json.dumps(row), flush=True)
            continue
        row = measure(args.model, tokens, args.iters, args.warmup, rank, world, dev, args.zipf,
                      args.graph, flush, args.fp8, args.replays, not args.no_verify)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
