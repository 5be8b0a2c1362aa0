"""In-tree build of the native library (`libpplx_kernels_b200.so`) for sm_100a.

Role parity: setup.py + csrc/CMakeLists.txt of the reference (setup.py:16-57,
csrc/CMakeLists.txt:1-77), which drive CMake/Ninja to produce
`libpplx_kernels.so` next to the Python package.  Here nvcc and g++ are invoked
directly: `.cu` files are compiled for exactly one target
(`-gencode arch=compute_100a,code=sm_100a`), host-only `.cpp` files with g++,
objects are cached under `pplx_kernels_b200/_build/` by content hash of the
source and every header it can include, and everything is linked into one shared
object inside the package so that it travels with a copy of the source tree.
nvcc cross-compiles, so the build needs no GPU.

Usage: ``python -m pplx_kernels_b200.build [--force] [--verbose] [--ptxas-info] [--cpp-tests]``.
"""

from __future__ import annotations

import argparse
import concurrent.futures
import hashlib
import os
import shlex
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "_build"
LIB_NAME = "libpplx_kernels_b200.so"
LIB_PATH = PKG_DIR / LIB_NAME

# Experiments: a library under another name (PPLX_B200_LIB_OUT, loaded through
# PPLX_B200_LIBRARY) built with extra nvcc flags (PPLX_B200_EXTRA_NVCC_FLAGS).
LIB_PATH = Path(os.environ.get("PPLX_B200_LIB_OUT", str(LIB_PATH)))
EXTRA_NVCC_FLAGS = shlex.split(os.environ.get("PPLX_B200_EXTRA_NVCC_FLAGS", ""))

CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _sources() -> list[Path]:
    out: list[Path] = []
    for sub in ("kernels", "runtime", "bindings"):
        d = CSRC / sub
        out += sorted(d.glob("*.cu")) + sorted(d.glob("*.cpp"))
    return out


def _headers() -> list[Path]:
    hs: list[Path] = []
    for ext in ("*.h", "*.cuh", "*.hpp", "*.inl"):
        hs += sorted(CSRC.rglob(ext))
    return hs


def _torch_paths() -> tuple[list[str], list[str]]:
    import torch.utils.cpp_extension as ce

    return ce.include_paths("cuda"), ce.library_paths("cuda")


def _needs_torch(src: Path) -> bool:
    return src.parent.name == "bindings"


def _digest(src: Path, header_blob: bytes, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    h.update(header_blob)
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _compile_cmd(src: Path, obj: Path, ptxas_info: bool) -> list[str]:
    includes = [f"-I{CUDA_HOME / 'include'}"]
    defines: list[str] = []
    if _needs_torch(src):
        import torch

        tinc, _ = _torch_paths()
        includes += [f"-I{p}" for p in tinc]
        includes.append(f"-I{sysconfig.get_paths()['include']}")
        defines += [
            "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        ]
    if src.suffix == ".cu":
        cmd = [NVCC, "-std=c++20", "-O3", *ARCH_FLAGS, "-lineinfo", "--expt-relaxed-constexpr",
               "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
               *includes, *defines, *EXTRA_NVCC_FLAGS]
        if ptxas_info:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", "-std=c++20", "-O2", "-fPIC", "-fvisibility=hidden", "-Wall",
               "-Wno-unused-function", *includes, *defines, "-c", str(src), "-o", str(obj)]
    return cmd


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compiles what changed and links the library; returns its path."""
    BUILD_DIR.mkdir(exist_ok=True)
    header_blob = b"".join(p.read_bytes() for p in _headers())
    jobs: list[tuple[Path, Path, list[str]]] = []
    objs: list[Path] = []
    for src in _sources():
        probe = _compile_cmd(src, Path("x.o"), ptxas_info)
        tag = _digest(src, header_blob, probe)
        obj = BUILD_DIR / f"{src.parent.name}_{src.stem}.{tag}.o"
        objs.append(obj)
        if force or not obj.exists():
            for stale in BUILD_DIR.glob(f"{src.parent.name}_{src.stem}.*.o"):
                stale.unlink()
            jobs.append((src, obj, _compile_cmd(src, obj, ptxas_info)))

    def run(job: tuple[Path, Path, list[str]]) -> str:
        src, obj, cmd = job
        if verbose:
            print(shlex.join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            if obj.exists():
                obj.unlink()
            raise RuntimeError(f"compiling {src} failed:\n{res.stdout}\n{res.stderr}")
        return f"[{src.name}]\n{res.stderr}" if (ptxas_info or verbose) and res.stderr else ""

    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            for log in ex.map(run, jobs):
                if log:
                    print(log, flush=True)

    stamp = BUILD_DIR / f"link.{LIB_PATH.name}.stamp"
    link_tag = hashlib.sha256(" ".join(sorted(o.name for o in objs)).encode()).hexdigest()
    if jobs or force or not LIB_PATH.exists() or not stamp.exists() or stamp.read_text() != link_tag:
        _, tlib = _torch_paths()
        cmd = ["g++", "-shared", "-o", str(LIB_PATH), *map(str, objs)]
        for p in tlib:
            cmd += [f"-L{p}", f"-Wl,-rpath,{p}"]
        cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart"]
        if verbose:
            print(shlex.join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        stamp.write_text(link_tag)
    return LIB_PATH


def build_cpp_tests(verbose: bool = False) -> list[Path]:
    """Builds the torch-free C++ executables (test_all_to_all, bench_all_to_all).

    Role parity: the WITH_TESTS / WITH_BENCHMARKS targets of the reference's CMake build
    (csrc/all_to_all/CMakeLists.txt:41-74), without MPI: the test runs its ranks on one GPU
    and the benchmark finds its peers through the socket bootstrap.
    """
    build()
    bin_dir = BUILD_DIR / "bin"
    bin_dir.mkdir(exist_ok=True)
    objs = [o for o in BUILD_DIR.glob("*.o") if not o.name.startswith("bindings_")]
    out = []
    for name in ("test_all_to_all", "bench_all_to_all"):
        exe = bin_dir / name
        cmd = ["g++", "-std=c++20", "-O2", f"-I{CUDA_HOME / 'include'}",
               str(CSRC / "tests" / f"{name}.cpp"), *map(str, objs), "-o", str(exe),
               f"-L{CUDA_HOME / 'lib64'}", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}", "-lcudart",
               "-lpthread", "-ldl"]
        if verbose:
            print(shlex.join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"building {name} failed:\n{res.stdout}\n{res.stderr}")
        out.append(exe)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true", help="recompile everything")
    ap.add_argument("--verbose", action="store_true", help="print the compiler commands")
    ap.add_argument("--ptxas-info", action="store_true",
                    help="pass -Xptxas -v and print register/shared-memory usage")
    ap.add_argument("--cpp-tests", action="store_true",
                    help="also build the C++ test and benchmark executables under _build/bin")
    args = ap.parse_args()
    path = build(force=args.force, verbose=args.verbose, ptxas_info=args.ptxas_info)
    print(path)
    if args.cpp_tests:
        for exe in build_cpp_tests(verbose=args.verbose):
            print(exe)


if __name__ == "__main__":
    sys.exit(main())
