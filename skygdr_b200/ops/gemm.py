"""bf16 GEMM on tcgen05 tensor cores (skygdr_b200/csrc/kernels/gemm_tcgen05.cu)."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .._ext import load
from .flow import new_status

_SM_COUNT: Dict[int, int] = {}


def _sms(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def pick_splits(M: int, N: int, K: int, sms: int, gated: bool = False) -> int:
    """Split-K factor for weight-streaming GEMMs: one CTA occupies one SM, so the CTA count should fill
    whole waves of ``sms``. Picks the factor (each split keeps at least 4 k-blocks of 64) whose last wave is
    fullest; ties go to the smaller factor."""
    C = load()
    ntok = C.gemm_pick_ntok(M, gated)
    tiles = ((N + 127) // 128) * ((M + ntok - 1) // ntok)
    kb = K // 64
    # Measured on B200: with more than half a wave of tiles, the prologue/epilogue each extra CTA pays
    # (barrier and TMEM set-up, pipeline fill, partial write + reduce) costs more than the idle SMs.
    if 2 * tiles > sms or M > 128:
        return 1
    best, best_eff = 1, 0.0
    for s in range(1, 17):
        if s > 1 and kb // s < 4:
            break
        per = (kb + s - 1) // s
        s_eff = (kb + per - 1) // per          # splits that actually get work
        ctas = tiles * s_eff
        waves = (ctas + sms - 1) // sms
        # time ~ waves * per (k-blocks streamed back to back by the busiest SM)
        eff = (tiles * kb) / (waves * per * sms)
        if s > 1:
            eff /= 1.0 + s_eff * ntok * 4.0 / K      # fp32 partials written and re-read, relative to the weight bytes
        if eff > best_eff + 0.03:
            best, best_eff = s, eff
    return best


class GemmWorkspace:
    """Scratch for split-K: fp32 partial tiles and per-tile counters, grown on demand, one per stream of use."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.ws = torch.empty(0, dtype=torch.float32, device=self.device)
        self.counters = torch.zeros(4096, dtype=torch.int32, device=self.device)
        self.status = new_status(self.device)

    def ensure(self, floats: int, counters: int):
        if self.ws.numel() < floats:
            self.ws = torch.empty(floats, dtype=torch.float32, device=self.device)
        if self.counters.numel() < counters:
            self.counters = torch.zeros(counters, dtype=torch.int32, device=self.device)


_WS: Dict[int, GemmWorkspace] = {}


def workspace_for(device) -> GemmWorkspace:
    idx = torch.device(device).index or 0
    if idx not in _WS:
        _WS[idx] = GemmWorkspace(device)
    return _WS[idx]


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, gated: bool = False,
         splits: Optional[int] = None, ws: Optional[GemmWorkspace] = None) -> torch.Tensor:
    """y = x @ w.T (w is [N][K]); gated: w is [2N][K] and y = silu(x @ w[:N].T) * (x @ w[N:].T)."""
    C = load()
    M, K = x.shape
    N = w.shape[0] // 2 if gated else w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if splits is None:
        splits = pick_splits(M, N, K, _sms(x.device), gated)
    ws = ws or workspace_for(x.device)
    if splits > 1:
        ws.ensure(C.gemm_workspace_floats(M, N, splits, gated), C.gemm_counter_count(M, N, gated))
        C.gemm(x, w, out, splits, gated, ws.ws, ws.counters, ws.status)
    else:
        C.gemm(x, w, out, 1, gated, None, None, ws.status)
    return out
