"""Throughput of the tcgen05 grouped GEMM on one GPU, against the measured cuBLAS peak.

    python -m pplx_kernels_b200.utils.bench_gemm --shape mixtral_up
    python -m pplx_kernels_b200.utils.bench_gemm --experts 8 --rows 512 --k 2048 --n 768 --swiglu
    python -m pplx_kernels_b200.utils.bench_gemm --shape mixtral_up --fp8

Times with CUDA events after warm-up, flushing L2 between iterations; prints one
JSON line with achieved TFLOP/s and the fraction of the measured bf16 peak
(MEASURED_PEAKS.json next to the repository root when present).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

from pplx_kernels_b200.ops.grouped_gemm import (
    grouped_gemm,
    grouped_gemm_fp8,
    quantize_weight_blocks,
)
from pplx_kernels_b200.ops.quant import per_token_block_quant

SHAPES = {
    # name: (experts, rows per expert, K, N, swiglu)
    "mixtral_up": (1, 1024, 4096, 14336, True),      # 512 tok/GPU x 8 GPUs x top-2 / 8 experts
    "mixtral_down": (1, 1024, 14336, 4096, False),
    "qwen3_up": (16, 128, 2048, 768, True),          # 256 tok/GPU, 128 experts, top-8, EP8
    "qwen3_down": (16, 128, 768, 2048, False),
    "deepseek_up": (32, 32, 7168, 2048, True),       # 128 tok/GPU, 256 experts, top-8, EP8
    "deepseek_down": (32, 32, 2048, 7168, False),
    "square_8k": (1, 8192, 8192, 8192, False),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", choices=sorted(SHAPES), default=None)
    ap.add_argument("--experts", type=int, default=1)
    ap.add_argument("--rows", type=int, default=1024)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--half-n", type=int, default=0, help="force the B half width (0 = choose)")
    ap.add_argument("--cta-pair", type=int, default=-1, help="1 = CTA pair, 0 = single, -1 = choose")
    ap.add_argument("--fp8", action="store_true",
                    help="block-scaled e4m3 kernel (with --swiglu its output is quantised too)")
    ap.add_argument("--pow2", action="store_true",
                    help="with --fp8: power-of-two scales, applied by the tensor cores")
    args = ap.parse_args()
    if args.shape:
        E, rows, K, N, swiglu = SHAPES[args.shape]
    else:
        E, rows, K, N, swiglu = args.experts, args.rows, args.k, args.n, args.swiglu

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    x = (torch.randn(E, rows, K, device=dev) * 0.5).to(torch.bfloat16)
    w = (torch.randn(E, (2 if swiglu else 1) * N, K, device=dev) * K ** -0.5).to(torch.bfloat16)
    counts = torch.full((E,), rows, dtype=torch.int32, device=dev)
    out = torch.empty(E, rows, N, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)

    def lib():
        # cuBLAS through torch on the same math (no fused activation), for context only
        for e in range(E):
            torch.matmul(x[e], w[e].t())

    if args.fp8:
        xq, sa = per_token_block_quant(x.view(E * rows, K), pow2=args.pow2)
        xq, sa = xq.view(E, rows, K), sa.view(E, rows, -1)
        wq, sw = quantize_weight_blocks(w, pow2=args.pow2)
        out8 = torch.empty(E, rows, N, dtype=torch.float8_e4m3fn, device=dev) if swiglu else out
        out8_scale = (torch.empty(E, rows, N // 128, dtype=torch.float32, device=dev)
                      if swiglu else None)

        def ours():
            grouped_gemm_fp8(xq, sa, wq, sw, counts, swiglu_quant=swiglu, out=out8,
                             out_scale=out8_scale, status=status, pow2_scales=args.pow2)
    else:
        def ours():
            grouped_gemm(x, w, counts, out=out, swiglu=swiglu, status=status,
                         expected_rows=E * rows, half_n=args.half_n, cta_pair=args.cta_pair)

    results = {}
    for name, fn in (("ours", ours), ("torch_matmul", lib)):
        times = []
        for it in range(args.warmup + args.iters):
            if not args.no_flush:
                flush.add_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                times.append(e0.elapsed_time(e1) * 1e3)
        results[name] = statistics.median(times)
    assert int(status.item()) == 0
    flops = 2.0 * E * rows * K * N * (2 if swiglu else 1)
    peak = None
    try:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            peak = json.load(f)["bf16_tflops"]
    except OSError:
        pass
    tf = flops / results["ours"] / 1e6
    print(json.dumps({
        "shape": {"experts": E, "rows": rows, "k": K, "n": N, "swiglu": swiglu},
        "dtype": ("fp8_e4m3, power-of-two block scales in hardware" if args.fp8 and args.pow2
                  else "fp8_e4m3 block-scaled" if args.fp8 else "bf16"),
        "us_p50": results["ours"],
        "tflops": tf,
        "frac_of_measured_bf16_peak": tf / peak if peak else None,
        "torch_matmul_us_p50": results["torch_matmul"],
        "torch_matmul_tflops": flops / results["torch_matmul"] / 1e6,
    }))


if __name__ == "__main__":
    main()
