"""Profiling driver for the kernels of the MoE layer on one GPU.

    python -m pplx_kernels_b200.utils.profile_moe --fused --iters 2            # bf16, fused
    python -m pplx_kernels_b200.utils.profile_moe --fp8 --iters 2              # fp8, composed
    python -m pplx_kernels_b200.utils.profile_moe --fp8 --fused --iters 2      # fp8, fused

runs a few forward passes of a one-rank layer whose activations and weights are larger than
the L2 but hold well under a gigabyte, so that it is the command to put under ``ncu`` with
``-k regex:<kernel>`` and a small ``-c``: the packed send (``dispatch_kernel``, fused), the
quantising send (``dispatch_kernel``, fp8 composed), the staging-fed and the peer-storing
expert GEMMs (``grouped_gemm_kernel`` / ``grouped_gemm_fp8_kernel``, fused) and the combine
reduction.  Prints CUDA-event times per pass.
"""

from __future__ import annotations

import argparse
import json

import torch

from pplx_kernels_b200.models.configs import MoEModelConfig
from pplx_kernels_b200.models.moe import MoELayer, MoELayerFP8
from pplx_kernels_b200.utils.testing import as_index_tensor, routing


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--fused", action="store_true")
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--pow2", action="store_true", help="fp8 with power-of-two (hardware) scales")
    args = ap.parse_args()

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = MoEModelConfig("profile", args.experts, args.topk, args.hidden, args.inter)
    extra = {"pow2_scales": True} if args.fp8 and args.pow2 else {}
    layer = (MoELayerFP8 if args.fp8 else MoELayer)(cfg, max_num_tokens=args.tokens, device=dev,
                                                    **extra)
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(args.tokens, cfg.hidden_dim, generator=gen).to(torch.bfloat16).to(dev)
    idx = as_index_tensor(routing(args.tokens, cfg.num_experts, cfg.experts_per_token, gen), dev)
    w = torch.softmax(torch.randn(args.tokens, cfg.experts_per_token, generator=gen), dim=-1).to(dev)
    out = torch.zeros(args.tokens, cfg.hidden_dim, dtype=torch.bfloat16, device=dev)
    times = []
    for _ in range(args.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        layer(x, idx, w, out=out, fused=args.fused)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    layer.check_status()
    layer.destroy()
    rows = args.tokens * cfg.experts_per_token
    print(json.dumps({
        "fp8": args.fp8, "fused": args.fused, "tokens": args.tokens, "rows": rows,
        "experts": cfg.num_experts, "hidden": cfg.hidden_dim, "inter": cfg.intermediate_dim,
        "layer_us": times,
        "gemm_flops": rows * 6 * cfg.hidden_dim * cfg.intermediate_dim,
        "weight_bytes": cfg.num_experts * 3 * cfg.hidden_dim * cfg.intermediate_dim
        * (1 if args.fp8 else 2),
    }))


if __name__ == "__main__":
    main()
