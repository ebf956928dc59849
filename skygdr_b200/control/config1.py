"""CPU-only control-loop experiment (two flows over a simulated shared link).

``kv_transfer`` (priority high, target 40 GB/s) gets Poisson requests
(20 req/s, seed 0) of 50-500 MB; ``kv_offload`` is a backlogged best-effort
flow; the link has 64 GB/s; the control window is 5 ms; the run lasts 10 s.
Arms follow the reference's case study (always-HIGH, always-LOW, controlled:
src/tools/pcie_case_study_analyze.py:140-154), plus the reference's ladder rule
at its own 100 ms rate for comparison.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List


@dataclass
class Config1:
    capacity_gbps: float = 64.0
    window_ms: float = 5.0
    tick_ms: float = 0.25
    duration_s: float = 10.0
    seed: int = 0
    rate_per_s: float = 20.0
    size_lo_mb: float = 50.0
    size_hi_mb: float = 500.0
    target_gbps: float = 40.0
    offload_offered_gbps: float = -1.0   # <0: backlogged at link rate
    arms: List[str] = field(default_factory=lambda: ["always_high", "always_low", "ladder_100ms", "ladder", "target_track"])


def _specs(ctl, cfg: Config1):
    kv = ctl.SimFlowSpec()
    kv.name, kv.priority, kv.target_gbps, kv.kind = "kv_transfer", 100, cfg.target_gbps, 0
    kv.set_arrivals(ctl.poisson_uniform(cfg.seed, cfg.rate_per_s, cfg.duration_s, cfg.size_lo_mb * 1e6,
                                        cfg.size_hi_mb * 1e6))
    off = ctl.SimFlowSpec()
    off.name, off.priority, off.target_gbps, off.kind = "kv_offload", 0, 0.0, 1
    off.backlogged = True
    off.offered_gbps = cfg.offload_offered_gbps
    return [kv, off]


def run_arm(cfg: Config1, arm: str):
    from . import ctl

    sc = ctl.SimConfig()
    sc.capacity_gbps, sc.window_ms, sc.tick_ms, sc.duration_s = cfg.capacity_gbps, cfg.window_ms, cfg.tick_ms, cfg.duration_s
    if arm == "always_high":
        sc.policy = "none"
    elif arm == "always_low":
        sc.policy = "static"
    elif arm == "ladder_100ms":
        sc.policy = "ladder"
        sc.policy_every_windows = max(1, int(round(100.0 / cfg.window_ms)))
    else:
        sc.policy = arm
    return ctl.run_simulation(sc, _specs(ctl, cfg))


def summarise(cfg: Config1, res) -> Dict[str, float]:
    from . import ctl

    ft = res.flow_times_ms(1)
    unfinished = sum(1 for r in res.requests if r.flow_id == 1 and r.finish_ms < 0)
    return {
        "requests": len(ft) + unfinished,
        "unfinished": unfinished,
        "flow_time_p50_ms": ctl.percentile(ft, 0.5) if ft else float("nan"),
        "flow_time_p99_ms": ctl.percentile(ft, 0.99) if ft else float("nan"),
        "flow_time_mean_ms": sum(ft) / len(ft) if ft else float("nan"),
        "kv_transfer_gb": res.bytes_moved[0] / 1e9,
        "offload_goodput_gbps": res.bytes_moved[1] / 1e9 / cfg.duration_s,
        "link_util_pct": 100.0 * res.link_bytes / (cfg.capacity_gbps * 1e9 * res.sim_time_s),
        "windows": res.windows,
    }


def run_config1(cfg: Config1 | None = None) -> Dict[str, Dict[str, float]]:
    cfg = cfg or Config1()
    return {arm: summarise(cfg, run_arm(cfg, arm)) for arm in cfg.arms}


def controller_csv(res) -> str:
    """Per-window budgets as CSV: the reference's controller columns that apply to a simulated link
    (src/tools/pcie_case_study_controller.py:250-271) plus flow, budget_bytes and window_id."""
    from . import ctl

    lines = ["t_ms,window_id,flow,mode,decision,budget_bytes,inst_gbps,smooth_gbps,backlog_bytes,link_util_pct"]
    for r in res.rows:
        lines.append(f"{r.t_ms:.3f},{r.window_id},{r.flow},{ctl.mode_name(r.mode)},{r.decision},{r.budget_bytes:.0f},"
                     f"{r.inst_gbps:.6f},{r.smooth_gbps:.6f},{r.backlog_bytes},{r.link_util_pct:.3f}")
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    import json

    print(json.dumps(run_config1(), indent=1))
