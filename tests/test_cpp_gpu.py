"""Runs the torch-free C++ test and benchmark executables on the GPU.

Counterpart of the reference's ctest target `AllToAllTest` (mpiexec -np 4
test_all_to_all, csrc/all_to_all/CMakeLists.txt:56-58); here the four ranks share one
GPU, so a single device is enough.
"""

import subprocess

import pytest

from pplx_kernels_b200.build import BUILD_DIR, build_cpp_tests

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def binaries():
    bin_dir = BUILD_DIR / "bin"
    if not (bin_dir / "test_all_to_all").exists() or not (bin_dir / "bench_all_to_all").exists():
        build_cpp_tests()
    return bin_dir


def test_cpp_host_classes(binaries):
    res = subprocess.run([str(binaries / "test_all_to_all")], capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failure(s)" in res.stdout


def test_cpp_benchmark_single_rank(binaries):
    res = subprocess.run([str(binaries / "bench_all_to_all"), "--tokens", "1,16", "--repeat", "2",
                          "--samples", "4", "--experts", "64", "--hidden", "2048", "--topk", "6"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "dispatch recv" in res.stdout and "combine send" in res.stdout


def test_cpp_benchmark_two_processes(binaries, tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    uid = tmp_path / "uid"
    procs = [subprocess.Popen([str(binaries / "bench_all_to_all"), "--world", "2", "--rank", str(r),
                               "--uid-file", str(uid), "--tokens", "8", "--repeat", "2",
                               "--samples", "4"],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "EP=2" in outs[0][0]
