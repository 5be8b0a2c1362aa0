"""Loads the native operator library and exposes it as ``_ops``.

Role parity: src/pplx_kernels/ops.py:8-16 of the reference, which calls
``torch.ops.load_library`` on the shared object shipped inside the package and
falls back to an empty namespace when loading fails.  Here a missing library is
built on the spot when a compiler is present, and a failure on a machine that
has a GPU is an error rather than a silent fallback: nothing in this package has
a Python implementation of the GPU kernels.

The library is loaded on the first use of an operator, not on import: helpers of
this package that are plain PyTorch (synthetic data, clock sampling, CPU
placement, the oracle) can then be imported by a process that must not map the
native library -- the benchmark arm that times the unmodified reference is one.
"""

from __future__ import annotations

import logging
import os
import types
from pathlib import Path

import torch

logger = logging.getLogger(__name__)

# PPLX_B200_LIBRARY points at another build of the library (an experiment, a debug build).
_LIB = Path(os.environ.get("PPLX_B200_LIBRARY") or
            Path(__file__).resolve().parent.parent / "libpplx_kernels_b200.so")


def _load() -> object:
    if not _LIB.exists() and os.environ.get("PPLX_B200_NO_AUTOBUILD", "0") != "1":
        try:
            from ..build import build

            build()
        except Exception as exn:  # pragma: no cover - depends on the toolchain
            logger.error("building %s failed: %s", _LIB.name, exn)
    try:
        torch.ops.load_library(str(_LIB))
        return torch.ops.pplx_kernels_b200
    except OSError as exn:
        if torch.cuda.is_available():
            raise RuntimeError(
                f"pplx_kernels_b200: cannot load {_LIB} on a machine with a GPU; "
                "run `python -m pplx_kernels_b200.build`"
            ) from exn
        logger.error("pplx_kernels_b200: native library unavailable (%s)", exn)
        return types.SimpleNamespace()


class _LazyOps:
    """Stands for ``torch.ops.pplx_kernels_b200``; loads the library on first attribute use."""

    _namespace: object | None = None

    def _resolve(self) -> object:
        if _LazyOps._namespace is None:
            _LazyOps._namespace = _load()
        return _LazyOps._namespace

    def __getattr__(self, name: str) -> object:
        return getattr(self._resolve(), name)


_ops = _LazyOps()


def is_loaded() -> bool:
    """True once the native library has been mapped into this process."""
    return _LazyOps._namespace is not None


def library_path() -> Path:
    return _LIB


def is_available() -> bool:
    return hasattr(_ops, "all_to_all_destroy")
