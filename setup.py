"""Packaging entry point.

Role parity: setup.py:16-103 of the reference, which drives CMake + Ninja from a
custom ``build_ext`` and ships ``libpplx_kernels.so`` as package data.  Here the
custom build step calls ``pplx_kernels_b200.build.build()``, which compiles the
CUDA sources for ``sm_100a`` with nvcc and links ``libpplx_kernels_b200.so`` into
the package directory (no CMake; nvcc cross-compiles, so no GPU is needed).

    python setup.py build_ext --inplace      # or: python -m pplx_kernels_b200.build
    python -m pip install --no-build-isolation .
"""

import importlib.util
from pathlib import Path

from setuptools import Extension, setup
from setuptools.command.build_ext import build_ext


class NvccBuild(build_ext):
    def run(self) -> None:
        spec = importlib.util.spec_from_file_location(
            "_pplx_b200_build", Path(__file__).parent / "pplx_kernels_b200" / "build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        lib = mod.build()
        if not self.inplace:
            dest = Path(self.build_lib) / "pplx_kernels_b200" / lib.name
            dest.parent.mkdir(parents=True, exist_ok=True)
            self.copy_file(str(lib), str(dest))


setup(
    ext_modules=[Extension("pplx_kernels_b200.libpplx_kernels_b200", sources=[])],
    cmdclass={"build_ext": NvccBuild},
    zip_safe=False,
)
