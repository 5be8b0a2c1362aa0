"""Expert-parallel MoE FFN layer: dispatch -> SwiGLU expert FFN -> combine.

``MoELayer`` owns one rank's slice of the experts (``num_experts // world_size``
experts, SwiGLU weights ``w13 = [gate; up]`` and ``w2``), an ``AllToAll`` and the
intermediate buffers, and runs

    tokens --dispatch--> per-expert rows --grouped GEMM + SwiGLU--> h
           --grouped GEMM--> y --combine (top-k weighted sum)--> tokens

on hand-written sm_100a kernels only: P2P dispatch/combine and the tcgen05
grouped GEMM.  The reference library stops at dispatch/combine and leaves the
expert computation to the caller (its tests fake it with ``x * 1.5``,
tests/test_all_to_all.py:248-250); this layer is what a caller such as an
inference engine builds on top.

All buffers are allocated once, no host synchronisation happens in ``forward``,
and the token count can be bounded on the device (``bound_m``), so a forward
pass can be captured in a CUDA graph.
"""

from __future__ import annotations

import torch

from ..all_to_all import AllToAll
from ..ops.grouped_gemm import grouped_gemm
from .configs import MoEModelConfig


def _random_expert_weights(cfg: MoEModelConfig, first_expert: int, count: int, seed: int,
                           std: float, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """N(0, std) weights of experts [first_expert, first_expert + count), generated on the
    device and seeded by GLOBAL expert id, so that every world size holds the same model."""
    H, I = cfg.hidden_dim, cfg.intermediate_dim
    gen = torch.Generator(device=device)
    w13 = torch.empty(count, 2 * I, H, dtype=torch.float32, device=device)
    w2 = torch.empty(count, H, I, dtype=torch.float32, device=device)
    for le in range(count):
        gen.manual_seed(seed * 100003 + first_expert + le)
        w13[le].normal_(0.0, std, generator=gen)
        w2[le].normal_(0.0, std, generator=gen)
    return w13, w2


class MoELayer:
    def __init__(self, cfg: MoEModelConfig, max_num_tokens: int, rank: int = 0,
                 world_size: int = 1, dp_size: int = 1, device: torch.device | None = None,
                 ata: AllToAll | None = None, seed: int = 0, group_name: str = "default",
                 init_std: float = 0.02) -> None:
        assert cfg.num_experts % world_size == 0
        self.cfg = cfg
        self.rank, self.world_size, self.dp_size = rank, world_size, dp_size
        self.max_num_tokens = max_num_tokens
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nle = cfg.num_experts // world_size
        self.rows = max_num_tokens * (world_size // dp_size)
        H, I = cfg.hidden_dim, cfg.intermediate_dim
        self.ata = ata or AllToAll.intranode(
            max_num_tokens, cfg.num_experts, cfg.experts_per_token, rank, world_size, dp_size,
            H, H * 2, 0, group_name=group_name)
        # Random-init weights of this rank's experts; every rank seeds by global expert id so
        # that any world size holds the same model.
        dev = self.device
        w13, w2 = _random_expert_weights(cfg, rank * self.nle, self.nle, seed, init_std, dev)
        self.w13 = w13.to(torch.bfloat16)  # [nle, 2I, H]
        self.w2 = w2.to(torch.bfloat16)    # [nle, H, I]
        self.counts = torch.zeros(self.nle, dtype=torch.int32, device=dev)
        self.expert_x = torch.zeros(self.nle, self.rows, H, dtype=torch.bfloat16, device=dev)
        self.h = torch.zeros(self.nle, self.rows, I, dtype=torch.bfloat16, device=dev)
        self.expert_y = torch.zeros(self.nle, self.rows, H, dtype=torch.bfloat16, device=dev)
        self.gemm_status = torch.zeros(1, dtype=torch.int32, device=dev)

    def forward(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                out: torch.Tensor | None = None, bound_m: torch.Tensor | None = None,
                fused: bool = True) -> torch.Tensor:
        """x: [m, hidden] bf16; indices: [m, top-k] uint32; weights: [m, top-k] fp32.

        ``fused=True`` runs four kernels: the packed dispatch send, the up projection fed
        from the staging arena as tokens land, the down projection whose epilogue stores to the
        tokens' home ranks, and the combine reduction.  ``fused=False`` runs the plain
        composition dispatch -> GEMM -> GEMM -> combine (six phases, two more passes over
        the activations).
        """
        if out is None:
            out = torch.empty(self.max_num_tokens, self.cfg.hidden_dim, dtype=torch.bfloat16,
                              device=self.device)
        # Rows this rank expects under uniform routing: steers the GEMM tile width only.
        expect = x.size(0) * self.cfg.experts_per_token * (self.world_size // self.dp_size) \
            // self.world_size
        if fused:
            self.ata.fused_dispatch(x, indices, bound_m)
            self.ata.fused_up(self.w13, self.h, self.counts, self.gemm_status, expect)
            self.ata.fused_down(self.h, self.w2, self.gemm_status, expect)
            self.ata.combine(out, indices, weights, self.expert_y, bound_m,
                             do_send=False, do_recv=True)
            return out
        self.ata.dispatch(self.counts, self.expert_x, None, x, None, indices, bound_m)
        grouped_gemm(self.expert_x, self.w13, self.counts, out=self.h, swiglu=True,
                     status=self.gemm_status, expected_rows=expect)
        grouped_gemm(self.h, self.w2, self.counts, out=self.expert_y, swiglu=False,
                     status=self.gemm_status, expected_rows=expect)
        self.ata.combine(out, indices, weights, self.expert_y, bound_m)
        return out

    __call__ = forward

    def check_status(self) -> None:
        self.ata.check_status()
        code = int(self.gemm_status.item())
        if code == 2:
            raise RuntimeError("pplx_kernels_b200: a grouped GEMM was told that its scales are "
                               "powers of two and found one that is not")
        if code != 0:
            raise RuntimeError("pplx_kernels_b200: a grouped GEMM pipeline wait ran out")

    def destroy(self) -> None:
        self.ata.destroy()


def moe_reference(x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                  w13: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """Plain PyTorch fp32 MoE FFN over ALL experts (w13: [E, 2I, H], w2: [E, H, I]).

    Intermediate roundings follow the kernels: h and y are rounded to bf16 before
    the next step, the top-k sum is accumulated in fp32.
    """
    m, _ = x.shape
    I = w2.size(2)
    out = torch.zeros(m, x.size(1), dtype=torch.float32, device=x.device)
    xf = x.to(torch.float32)
    idx = indices.to(torch.int64)
    for k in range(idx.size(1)):
        for e in idx[:, k].unique().tolist():
            sel = (idx[:, k] == e).nonzero().flatten()
            y = xf[sel] @ w13[e].to(torch.float32).t()
            h = (torch.nn.functional.silu(y[:, :I]) * y[:, I:]).to(torch.bfloat16).to(torch.float32)
            o = (h @ w2[e].to(torch.float32).t()).to(torch.bfloat16).to(torch.float32)
            out[sel] += o * weights[sel, k : k + 1].to(torch.float32)
    return out


class MoELayerFP8:
    """The same expert FFN with block-scaled fp8 weights and activations.

    Tokens enter as bf16; ``dispatch_quant`` converts them to e4m3 with one fp32 scale per 128
    columns while sending; the up projection runs on ``kind::f8f6f4`` tensor cores with the
    weights' 128 x 128 block scales, applies SwiGLU and re-quantises its result in its
    epilogue; the down projection produces bf16 rows for ``combine``.  (DeepSeek-V3 / Qwen3
    style fp8 inference.)
    """

    def __init__(self, cfg: MoEModelConfig, max_num_tokens: int, rank: int = 0,
                 world_size: int = 1, dp_size: int = 1, device: torch.device | None = None,
                 seed: int = 0, group_name: str = "default", init_std: float = 0.02,
                 ata: AllToAll | None = None, pow2_scales: bool = False) -> None:
        """``pow2_scales``: every scale (weights at load, activations in the quantising send and
        in the up projection's epilogue) is a power of two, which lets the tensor cores apply
        them (``kind::mxf8f6f4.block_scale``) instead of the CUDA cores: about 1.5x the GEMM
        rate on compute-bound shapes, for at most one bit less of headroom per block."""
        from ..ops.grouped_gemm import quantize_weight_blocks

        assert cfg.num_experts % world_size == 0 and cfg.intermediate_dim % 128 == 0
        self.pow2_scales = pow2_scales
        self.cfg = cfg
        self.rank, self.world_size, self.dp_size = rank, world_size, dp_size
        self.max_num_tokens = max_num_tokens
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nle = cfg.num_experts // world_size
        self.rows = max_num_tokens * (world_size // dp_size)
        H, I = cfg.hidden_dim, cfg.intermediate_dim
        nscale = (H + 127) // 128
        self.ata = ata or AllToAll.intranode(
            max_num_tokens, cfg.num_experts, cfg.experts_per_token, rank, world_size, dp_size,
            H, H, nscale * 4, group_name=group_name)
        dev = self.device
        w13, w2 = _random_expert_weights(cfg, rank * self.nle, self.nle, seed, init_std, dev)
        self.ata.set_power_of_two_scales(pow2_scales)
        self.w13_q, self.w13_s = quantize_weight_blocks(w13, pow2=pow2_scales)
        self.w2_q, self.w2_s = quantize_weight_blocks(w2, pow2=pow2_scales)
        del w13, w2
        self.counts = torch.zeros(self.nle, dtype=torch.int32, device=dev)
        self.expert_x = torch.zeros(self.nle, self.rows, H, dtype=torch.uint8,
                                    device=dev).view(torch.float8_e4m3fn)
        self.expert_scale = torch.zeros(self.nle, self.rows, nscale, device=dev)
        self.h = torch.zeros(self.nle, self.rows, I, dtype=torch.uint8,
                             device=dev).view(torch.float8_e4m3fn)
        self.h_scale = torch.zeros(self.nle, self.rows, I // 128, device=dev)
        self.expert_y = torch.zeros(self.nle, self.rows, H, dtype=torch.bfloat16, device=dev)
        self.gemm_status = torch.zeros(1, dtype=torch.int32, device=dev)

    def forward(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                out: torch.Tensor | None = None, bound_m: torch.Tensor | None = None,
                fused: bool = False) -> torch.Tensor:
        """``fused=True``: quantising packed send, fp8 up projection fed from the staging
        arena (rows and scales) as tokens land, fp8 down projection whose epilogue stores to
        the tokens' home ranks, combine reduction -- four kernels.  ``fused=False``: the
        composition dispatch_quant -> GEMM -> GEMM -> combine."""
        from ..ops.grouped_gemm import grouped_gemm_fp8

        if out is None:
            out = torch.empty(self.max_num_tokens, self.cfg.hidden_dim, dtype=torch.bfloat16,
                              device=self.device)
        if fused:
            self.ata.fused_dispatch(x, indices, bound_m, quantize=True)
            self.ata.fused_up_fp8(self.w13_q, self.w13_s, self.h, self.h_scale, self.counts,
                                  self.gemm_status)
            self.ata.fused_down_fp8(self.h, self.h_scale, self.w2_q, self.w2_s, self.gemm_status)
            self.ata.combine(out, indices, weights, self.expert_y, bound_m,
                             do_send=False, do_recv=True)
            return out
        self.ata.dispatch_quant(self.counts, self.expert_x, self.expert_scale, x, indices, bound_m)
        grouped_gemm_fp8(self.expert_x, self.expert_scale, self.w13_q, self.w13_s, self.counts,
                         swiglu_quant=True, out=self.h, out_scale=self.h_scale,
                         status=self.gemm_status, pow2_scales=self.pow2_scales)
        grouped_gemm_fp8(self.h, self.h_scale, self.w2_q, self.w2_s, self.counts,
                         out=self.expert_y, status=self.gemm_status,
                         pow2_scales=self.pow2_scales)
        self.ata.combine(out, indices, weights, self.expert_y, bound_m)
        return out

    __call__ = forward

    def dequantized_weights(self) -> tuple[torch.Tensor, torch.Tensor]:
        """fp32 views of this rank's weights as the kernels see them (for references)."""
        def deq(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
            full = s.repeat_interleave(128, dim=1)[:, : q.size(1)].repeat_interleave(128, dim=2)
            return q.to(torch.float32) * full[:, :, : q.size(2)]

        return deq(self.w13_q, self.w13_s), deq(self.w2_q, self.w2_s)

    def check_status(self) -> None:
        self.ata.check_status()
        code = int(self.gemm_status.item())
        if code == 2:
            raise RuntimeError("pplx_kernels_b200: a grouped GEMM was told that its scales are "
                               "powers of two and found one that is not")
        if code != 0:
            raise RuntimeError("pplx_kernels_b200: a grouped GEMM pipeline wait ran out")

    def destroy(self) -> None:
        self.ata.destroy()


def moe_reference_fp8(x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                      w13: torch.Tensor, w2: torch.Tensor, pow2: bool = False) -> torch.Tensor:
    """Plain PyTorch statement of the fp8 layer: activations pass through the same block
    quantisation as in the kernels (before each GEMM), weights are given de-quantised."""
    from ..ops.quant import block_dequant, per_token_block_quant

    m = x.size(0)
    I = w2.size(2)
    xq = block_dequant(*per_token_block_quant(x.cpu(), pow2=pow2)).to(x.device)
    out = torch.zeros(m, x.size(1), dtype=torch.float32, device=x.device)
    idx = indices.to(torch.int64)
    for k in range(idx.size(1)):
        for e in idx[:, k].unique().tolist():
            sel = (idx[:, k] == e).nonzero().flatten()
            y = xq[sel] @ w13[e].t()
            h = torch.nn.functional.silu(y[:, :I]) * y[:, I:]
            h = block_dequant(*per_token_block_quant(h.cpu(), pow2=pow2)).to(x.device)
            o = (h @ w2[e].t()).to(torch.bfloat16).to(torch.float32)
            out[sel] += o * weights[sel, k : k + 1].to(torch.float32)
    return out
