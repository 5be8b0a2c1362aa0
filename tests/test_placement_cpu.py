import pytest

from pplx_kernels_b200.models.configs import CONFIGS, MIXTRAL_8X7B
from pplx_kernels_b200.parallel import EPLayout


def test_block_partition_and_dp_groups():
    lay = EPLayout(num_experts=8, world_size=4, dp_size=2)
    assert lay.num_local_experts == 2 and lay.num_dp_groups == 2
    assert [lay.owner(e) for e in range(8)] == [0, 0, 1, 1, 2, 2, 3, 3]
    assert [lay.local_index(e) for e in range(8)] == [0, 1] * 4
    assert list(lay.local_experts(3)) == [6, 7]
    assert lay.dp_group(3) == 1 and list(lay.group_ranks(1)) == [2, 3]
    # tokens of a group alternate between its ranks
    assert [lay.sender_of(1, t) for t in range(4)] == [2, 3, 2, 3]
    assert lay.rows_per_expert(10) == 20


def test_invalid_layouts_are_rejected():
    with pytest.raises(ValueError):
        EPLayout(num_experts=7, world_size=2)
    with pytest.raises(ValueError):
        EPLayout(num_experts=8, world_size=4, dp_size=3)


def test_model_configs():
    assert set(CONFIGS) >= {"mixtral-8x7b", "qwen3-30b-a3b", "deepseek-v3"}
    assert MIXTRAL_8X7B.flops_per_token() == 2 * 3 * 4096 * 14336 * 2
