"""Loads the native operator library and exposes it as ``_ops``.

Role parity: src/pplx_kernels/ops.py:8-16 of the reference, which calls
``torch.ops.load_library`` on the shared object shipped inside the package and
falls back to an empty namespace when loading fails.  Here a missing library is
built on the spot when a compiler is present, and a failure on a machine that
has a GPU is an error rather than a silent fallback: nothing in this package has
a Python implementation of the GPU kernels.
"""

from __future__ import annotations

import logging
import os
import types
from pathlib import Path

import torch

logger = logging.getLogger(__name__)

_LIB = Path(__file__).resolve().parent.parent / "libpplx_kernels_b200.so"


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


_ops = _load()


def library_path() -> Path:
    return _LIB


def is_available() -> bool:
    return hasattr(_ops, "all_to_all_destroy")
