"""bf16 GEMM on tcgen05 tensor cores (skygdr_b200/csrc/kernels/gemm_tcgen05.cu)."""
from __future__ import annotations

from dataclasses import dataclass
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
    """Split-K factor for the default token tile (kept for callers that do not choose the tile)."""
    return pick_config(M, N, K, sms, gated, fixed_ntok=load().gemm_pick_ntok(M, gated))[1]


@dataclass(frozen=True)
class GemmCostModel:
    """Constants of the tile/split chooser (microseconds, bytes per microsecond)."""
    fixed_alone: float          # prologue + epilogue of a CTA that has its SM to itself
    fixed_shared: float         # ... of a CTA that shares the SM with another
    rate_alone: float           # stream rate of a CTA alone on its SM
    rate_shared: float          # ... of each of two co-resident CTAs
    two_per_sm: bool            # count two CTA slots per SM for small pipeline stages
    part_write_rate: float      # a split writes its fp32 partial at this rate (inf = free)
    part_read_rate: float       # the last CTA of a tile re-reads all partials at this rate
    hbm_rate: float = 5.5e6


# Fitted to a measured sweep on B200 of the decoder's GEMM shapes at 1, 2, 4 and 8-way tensor parallelism (16 to 128 token rows):
# every shape as a chain of launches inside a CUDA graph, each launch on its own copy of the weights (cold in HBM), token tiles
# 16-128 and 1-16 splits. Summed over the 16 shapes the chosen configurations are 3.4 us slower than the best measured ones.
STANDALONE = GemmCostModel(1.56, 1.75, 36.4e3, 57.4e3, True, float("inf"), 26.2e3, hbm_rate=5.76e6)
# The GEMMs that wait for an all-gather (reduce-scatter + all-gather form of the tensor-parallel step) run one CTA per SM and
# raise arrivals per token tile, so fewer, larger CTAs win there. These are the constants under which that form was tuned end
# to end (TP 2 / 4 / 8).
FUSED_TP = GemmCostModel(6.0, 6.0, 55e3, 55e3, False, 100e3, 200e3)


_TUNED: Optional[Dict[str, list]] = None


def tuned_config(M: int, N: int, K: int, gated: bool) -> Optional[Tuple[int, int, bool]]:
    """(token tile, splits, cluster) measured fastest for exactly this shape by benchmarks/gemm_tune.py, or None. The table
    (ops/gemm_tuned.json) holds the decoder's projections at the tensor-parallel degrees and batch sizes of the benchmark."""
    global _TUNED
    if _TUNED is None:
        import json
        import os

        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gemm_tuned.json")
        try:
            _TUNED = json.load(open(path))["table"]
        except (OSError, ValueError, KeyError):
            _TUNED = {}
    e = _TUNED.get(f"{M},{N},{K},{int(gated)}")
    return (int(e[0]), int(e[1]), bool(e[2])) if e else None


def choose_config(M: int, N: int, K: int, sms: int, gated: bool = False) -> Tuple[int, int, bool]:
    """(token tile, splits, cluster) for a decode GEMM: the measured best where the shape was tuned, the cost model otherwise."""
    t = tuned_config(M, N, K, gated)
    if t:
        return t
    ntok, splits = pick_config(M, N, K, sms, gated)
    return ntok, splits, False


def pick_config(M: int, N: int, K: int, sms: int, gated: bool = False, fixed_ntok: int = 0,
                model: GemmCostModel = STANDALONE) -> Tuple[int, int]:
    """(token tile, split-K factor) for y[M][N] = x[M][K] w[N][K]^T with small M, from the cost model.

    The time is about waves x (fixed cost per CTA + bytes per CTA / stream rate of a CTA), bounded below by total bytes
    over the HBM rate; a split adds its fp32 partial (written, then re-read by the last CTA of the tile). A pipeline of
    small stages fits two CTAs on an SM, which then share the SM's stream rate."""
    wrows = 2 if gated else 1
    kb = K // 64
    cands = [fixed_ntok] if fixed_ntok else [n for n in (16, 32, 64, 128, 256) if n >= 16 and (n < 2 * M or n == 16) and not (gated and n > 128)]
    best, best_t = (cands[-1], 1), float("inf")
    tiles_n = (N + 127) // 128
    for ntok in cands:
        tiles_m = (M + ntok - 1) // ntok
        for s in range(1, 17):
            if s > 1 and kb // s < 4:
                break
            per = (kb + s - 1) // s
            s_eff = (kb + per - 1) // per
            if s_eff != s and model.two_per_sm:
                continue                               # the same partition as a smaller s
            ctas = tiles_n * tiles_m * s_eff
            stage = 128 * 64 * 2 * wrows + ntok * 64 * 2
            two = model.two_per_sm and 3 * stage <= 104 * 1024     # the kernel fits two CTAs per SM for small stages
            slots = sms * (2 if two else 1)
            waves = (ctas + slots - 1) // slots
            shared = two and ctas > sms                # two co-resident CTAs share the SM's stream rate
            part = ntok * 128 * 4 * wrows
            split_cost = part / model.part_write_rate + 1.0 + s_eff * part / model.part_read_rate if s_eff > 1 else 0.0
            t_cta = (model.fixed_shared if shared else model.fixed_alone) + per * stage / (model.rate_shared if shared else model.rate_alone) + split_cost
            hbm = (tiles_n * 128 * K * 2 * wrows + M * K * 2) / model.hbm_rate
            t = max(waves * t_cta, hbm)
            if t < best_t * 0.92:                      # simpler shapes come first; a rival must be clearly better
                best, best_t = (ntok, s_eff), t
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


def wide_tiles_pay(M: int, N: int, K: int, sms: int, gated: bool, ntok: int = 0) -> bool:
    """Whether the persistent form should walk tiles of 256 rows x 256 tokens instead of 128 x 256. The wide tile's main loop is
    about a fifth faster (two MMAs per token operand: a third less traffic from L2 per MMA), but its epilogue is not overlapped
    (7 % of a tile at K = 4096, less at larger K) and there are half as many tiles to spread over the SMs; it pays when its waves
    of tiles are not much emptier than the narrow form's. Measured on B200 (TFLOP/s, wide against narrow): 2048 x 4096 x 4096
    1220 / 1137, 4096 x 4096 x 4096 1315 / 1303, 8192 x 4096 x 4096 1362 / 1391, 8192 x 6144 x 4096 1351 / 1329,
    8192 x 4096 x 12288 1420 / 1333; gated (a gate and an up block per 256 tokens against 128-token tiles) 8192 x 12288 x 4096
    1463 / 1236, 4096 tokens 1505 / 1335, 2048 tokens 1418 / 1270. The rule below picks the faster one in all eight."""
    if ntok == 128 or (not gated and N % 256):
        return False
    tm = (M + 255) // 256
    if gated:       # narrow: 128 outputs x 128 tokens per tile; wide: 128 outputs x 256 tokens
        narrow, wide = ((N + 127) // 128) * ((M + 127) // 128), ((N + 127) // 128) * tm
    else:
        narrow, wide = (N // 128) * tm, (N // 256) * tm

    def fill(tiles):
        return tiles / (sms * ((tiles + sms - 1) // sms))

    speedup = 1.2 / (1.0 + 0.07 * 4096.0 / K)
    return speedup * fill(wide) > fill(narrow)


def gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, gated: bool = False,
         splits: Optional[int] = None, ws: Optional[GemmWorkspace] = None, ntok: int = 0, persistent: Optional[bool] = None,
         cluster: bool = False) -> torch.Tensor:  # noqa: C901
    """y = x @ w.T (w is [N][K]); gated: w is [2N][K] and y = silu(x @ w[:N].T) * (x @ w[N:].T).

    Few tokens (M <= 256, decode): one CTA per output tile with split-K, tile and split chosen by ``pick_config``.
    Many tokens (prefill): the persistent form, one CTA per SM walking tiles of 256 tokens (128 when gated) with two
    accumulators in TMEM, so that a tile's epilogue overlaps the next tile's MMAs, or tiles of 256 rows x 256 tokens where
    ``wide_tiles_pay`` says so. ``persistent`` overrides the choice (False = one tile per CTA at any M, kept for comparison;
    "wide" / "narrow" = that tile). ``cluster`` (2 to 8 splits): the splits of a tile run as a
    thread-block cluster and sum their partial accumulators through distributed shared memory instead of a workspace."""
    C = load()
    M, K = x.shape
    N = w.shape[0] // 2 if gated else w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    ws = ws or workspace_for(x.device)
    if persistent is None:
        persistent = M > 256 and splits in (None, 1)
    if persistent:
        wide = persistent == "wide" or (persistent is True and wide_tiles_pay(M, N, K, _sms(x.device), gated, ntok))
        C.gemm(x, w, out, 1, gated, None, None, ws.status, 256 if wide else (128 if (gated or ntok == 128) else 256), 2 if wide else 1)
        return out
    if splits is None:
        if ntok == 0 and M <= 256:
            ntok, splits, cluster = choose_config(M, N, K, _sms(x.device), gated)
        else:
            splits = 1 if M > 256 else pick_config(M, N, K, _sms(x.device), gated, fixed_ntok=ntok)[1]
    if splits > 1 and cluster:
        assert splits <= 8, "a cluster holds at most 8 CTAs"
        C.gemm(x, w, out, splits, gated, None, None, ws.status, ntok, False, True)
    elif splits > 1:
        ws.ensure(C.gemm_workspace_floats(M, N, splits, gated, ntok), C.gemm_counter_count(M, N, gated, ntok))
        C.gemm(x, w, out, splits, gated, ws.ws, ws.counters, ws.status, ntok)
    else:
        C.gemm(x, w, out, 1, gated, None, None, ws.status, ntok)
    return out
