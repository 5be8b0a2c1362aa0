"""Who owns which expert, which rank sends which token."""

from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class EPLayout:
    num_experts: int
    world_size: int
    dp_size: int = 1

    def __post_init__(self) -> None:
        if self.num_experts <= 0:
            raise ValueError("num_experts must be positive")
        if self.world_size % self.dp_size:
            raise ValueError("dp_size must divide world_size")

    @property
    def num_local_experts(self) -> int:
        """Expert slots per rank: blocks of ceil(E / W); the last rank(s) own fewer real ones."""
        return -(-self.num_experts // self.world_size)

    @property
    def num_dp_groups(self) -> int:
        return self.world_size // self.dp_size

    def owner(self, expert: int) -> int:
        """Rank that holds `expert`."""
        return expert // self.num_local_experts

    def local_index(self, expert: int) -> int:
        return expert % self.num_local_experts

    def local_experts(self, rank: int) -> range:
        n = self.num_local_experts
        return range(min(rank * n, self.num_experts), min((rank + 1) * n, self.num_experts))

    def dp_group(self, rank: int) -> int:
        return rank // self.dp_size

    def group_ranks(self, group: int) -> range:
        return range(group * self.dp_size, (group + 1) * self.dp_size)

    def sender_of(self, group: int, token: int) -> int:
        """Rank of `group` that puts `token` on the wire (the group splits the send work)."""
        return group * self.dp_size + token % self.dp_size

    def rows_per_expert(self, max_num_tokens: int) -> int:
        """Capacity of out_expert_x / expert_y along dim 1."""
        return max_num_tokens * self.num_dp_groups
