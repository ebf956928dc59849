"""NVTX ranges for timelines (nsys): no-ops unless SKYGDR_NVTX=1, so the hot path pays nothing by default.

The reference documents `nsys profile -t cuda,nvtx` (llm_problem_analysis/README.md:1003-1021) but emits no ranges."""
from __future__ import annotations

import contextlib
import os

_ON = os.environ.get("SKYGDR_NVTX", "0") == "1"


@contextlib.contextmanager
def nvtx_range(name: str):
    if not _ON:
        yield
        return
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
