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
        EPLayout(num_experts=0, world_size=2)
    with pytest.raises(ValueError):
        EPLayout(num_experts=8, world_size=4, dp_size=3)


def test_uneven_expert_count_uses_blocks_of_the_ceiling():
    lay = EPLayout(num_experts=10, world_size=4)
    assert lay.num_local_experts == 3
    assert [lay.owner(e) for e in range(10)] == [0, 0, 0, 1, 1, 1, 2, 2, 2, 3]
    assert list(lay.local_experts(3)) == [9]
    lay = EPLayout(num_experts=5, world_size=4)
    assert lay.num_local_experts == 2 and list(lay.local_experts(3)) == []


def test_model_configs():
    assert set(CONFIGS) >= {"mixtral-8x7b", "qwen3-30b-a3b", "deepseek-v3"}
    assert MIXTRAL_8X7B.flops_per_token() == 2 * 3 * 4096 * 14336 * 2


def test_cpulist_parsing_and_device_lookup(tmp_path):
    from pplx_kernels_b200.parallel import affinity

    assert affinity.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert affinity.parse_cpulist("") == set()
    assert affinity.pci_address(0, 0x1B, 0) == "0000:1b:00.0"

    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "local_cpulist").write_text("4-7\n")
    assert affinity.device_local_cpus("0000:1b:00.0", tmp_path) == {4, 5, 6, 7}

    # no local_cpulist: fall back to the node's cpulist
    dev2 = tmp_path / "bus" / "pci" / "devices" / "0000:9b:00.0"
    dev2.mkdir(parents=True)
    (dev2 / "numa_node").write_text("1\n")
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("56-59\n")
    assert affinity.device_local_cpus("0000:9b:00.0", tmp_path) == {56, 57, 58, 59}

    # unknown device, or a node of -1: nothing to bind to
    assert affinity.device_local_cpus("0000:ff:00.0", tmp_path) == set()
    (dev2 / "numa_node").write_text("-1\n")
    assert affinity.device_local_cpus("0000:9b:00.0", tmp_path) == set()


def test_bind_without_a_gpu_is_a_no_op():
    import os

    from pplx_kernels_b200.parallel import affinity

    before = os.sched_getaffinity(0)
    info = affinity.bind_to_device_numa_node(0)
    assert info["bound"] is False and info["reason"]
    assert os.sched_getaffinity(0) == before


def test_logging_prefix_and_routing_description(capsys):
    import logging

    import torch

    from pplx_kernels_b200.utils.logging_utils import describe_routing, init_logging

    log = init_logging(rank=3, level="DEBUG")
    log.debug("hello")
    logging.shutdown()
    err = capsys.readouterr().err
    assert "[rank 3]" in err and "hello" in err
    text = describe_routing(torch.tensor([[0, 5], [9, 5]]), num_experts=10, world_size=4)
    assert text.splitlines()[0] == "rank 0: 1 rows, per expert [1, 0, 0]"
    assert text.splitlines()[1] == "rank 1: 2 rows, per expert [0, 0, 2]"
    assert text.splitlines()[3] == "rank 3: 1 rows, per expert [1]"
