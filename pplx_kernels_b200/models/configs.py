"""MoE layer shapes of the model families this package is benchmarked on.

The reference ships no model code; its benchmark only names two all-to-all
shapes (tests/bench_all_to_all.py:255-272: DeepSeek-V2-Lite and R1).  The fused
MoE layer here needs the expert FFN sizes as well.
"""

from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class MoEModelConfig:
    name: str
    num_experts: int
    experts_per_token: int
    hidden_dim: int
    intermediate_dim: int  # per-expert FFN width (SwiGLU: gate and up are this wide each)

    def flops_per_token(self) -> int:
        """Expert FFN FLOPs for one token (gate + up + down, top-k experts)."""
        return 2 * 3 * self.hidden_dim * self.intermediate_dim * self.experts_per_token


MIXTRAL_8X7B = MoEModelConfig("mixtral-8x7b", 8, 2, 4096, 14336)
QWEN3_30B_A3B = MoEModelConfig("qwen3-30b-a3b", 128, 8, 2048, 768)
DEEPSEEK_V3 = MoEModelConfig("deepseek-v3", 256, 8, 7168, 2048)
DEEPSEEK_V2_LITE = MoEModelConfig("deepseek-v2-lite", 64, 6, 2048, 1408)
TINY = MoEModelConfig("tiny", 8, 2, 256, 384)

CONFIGS = {c.name: c for c in (MIXTRAL_8X7B, QWEN3_30B_A3B, DEEPSEEK_V3, DEEPSEEK_V2_LITE, TINY)}
