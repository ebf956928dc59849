"""Loader of the CUDA extension ``skygdr_b200._C``.

The extension lives in the package directory. It is built on demand where
nvcc exists. On a machine with a GPU a missing or unloadable extension is an
error, never a silent fallback to PyTorch ops.
"""
from __future__ import annotations

import importlib
import shutil

_C = None
_ERR = None


def load():
    global _C, _ERR
    if _C is not None:
        return _C
    import torch  # the extension links against libtorch; import it first

    try:
        _C = importlib.import_module("skygdr_b200._C")
        return _C
    except ImportError as exc:
        _ERR = exc
    if shutil.which("nvcc") is not None:
        from . import build

        build.build_cuda()
        importlib.invalidate_caches()
        _C = importlib.import_module("skygdr_b200._C")
        return _C
    raise RuntimeError(f"skygdr_b200._C is not built and nvcc is not available: {_ERR}")


def available() -> bool:
    try:
        load()
        return True
    except Exception:
        return False
