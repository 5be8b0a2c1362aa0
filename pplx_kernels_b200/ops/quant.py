"""Block-scaled fp8 (e4m3) quantisation in plain PyTorch: the oracle for the
quantisation that ``AllToAll.dispatch_quant`` fuses into the send.

One fp32 scale per ``block`` (128) consecutive columns of a row:
``scale = max(amax, 1e-4) / 448`` and ``q = round_to_e4m3(x * (448 / max(amax, 1e-4)))``.
"""

from __future__ import annotations

import torch


def per_token_block_quant(x: torch.Tensor, block: int = 128,
                          pow2: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """x: [m, hidden] -> (q [m, hidden] float8_e4m3fn, scale [m, ceil(hidden / block)] fp32).
    With ``pow2`` the scale is the smallest power of two that is not below ``amax / 448``."""
    m, hidden = x.shape
    nblk = (hidden + block - 1) // block
    xf = x.to(torch.float32)
    pad = nblk * block - hidden
    if pad:
        xf = torch.nn.functional.pad(xf, (0, pad))
    v = xf.view(m, nblk, block)
    amax = v.abs().amax(dim=2).clamp(min=1e-4)
    if pow2:
        scale = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
        q = (v / scale.unsqueeze(2)).clamp(-448.0, 448.0)
    else:
        scale = amax / 448.0
        q = (v * (448.0 / amax).unsqueeze(2)).clamp(-448.0, 448.0)
    q = q.to(torch.float8_e4m3fn).view(m, nblk * block)[:, :hidden]
    return q.contiguous(), scale.contiguous()


def block_dequant(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Inverse of ``per_token_block_quant`` in fp32."""
    hidden = q.size(-1)
    s = scale.repeat_interleave(block, dim=-1)[..., :hidden]
    return q.to(torch.float32) * s
