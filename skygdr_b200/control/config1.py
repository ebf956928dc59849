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


def run_live(cfg: Config1 | None = None, policy: str = "target_track", time_scale: float = 1.0) -> Dict[str, float]:
    """The same experiment against the real daemon process, in real time.

    ``fabricd`` runs as its own process with its own window timer; this process registers the two flows over TCP the way
    a client does (REGISTER, lease renewals), maps their credit pages, and plays the data paths and the shared link: every
    ~0.25 ms of wall time it shares the elapsed link capacity max-min between the flows, never moving a flow beyond its grant,
    and publishes consumed / completed / backlog bytes in the pages, which is all the daemon ever sees. Nothing here calls
    into the daemon's code: what is measured is the deployed control loop (socket, timer thread, shared pages, policy).
    ``time_scale`` < 1 shortens the run (duration and request sizes shrink together) for tests."""
    import time

    from . import FabricClient, FabricDaemon, ctl

    cfg = cfg or Config1()
    dur = cfg.duration_s * time_scale
    arrivals = [(t * time_scale, int(b * time_scale)) for t, b in ctl.poisson_uniform(cfg.seed, cfg.rate_per_s / time_scale, cfg.duration_s * time_scale,
                                                                                 cfg.size_lo_mb * 1e6 / time_scale, cfg.size_hi_mb * 1e6 / time_scale)] \
        if time_scale != 1.0 else list(ctl.poisson_uniform(cfg.seed, cfg.rate_per_s, cfg.duration_s, cfg.size_lo_mb * 1e6, cfg.size_hi_mb * 1e6))
    cap = cfg.capacity_gbps * 1e9
    with FabricDaemon(policy=policy, window_us=int(cfg.window_ms * 1000), capacity_gbps=cfg.capacity_gbps, lease_ms=2000) as d, \
            FabricClient(port=d.port) as c:
        kv = c.register("kv_transfer", "high", cfg.target_gbps)
        off = c.register("kv_offload", "besteffort", 0.0)
        flows = [kv, off]
        consumed = [0, 0]
        queue: List[List[float]] = []            # [remaining bytes, arrival time]
        done_ms: List[float] = []
        next_arrival = 0
        t0 = time.perf_counter()
        t_prev, t_renew = 0.0, 0.0
        while True:
            time.sleep(cfg.tick_ms * 1e-3)
            now = time.perf_counter() - t0
            dt, t_prev = now - t_prev, now
            while next_arrival < len(arrivals) and arrivals[next_arrival][0] <= now:
                queue.append([float(arrivals[next_arrival][1]), arrivals[next_arrival][0]])
                next_arrival += 1
            if now > dur and not queue:
                break
            if now > dur + 5.0:
                break                                # a stuck run ends with unfinished requests instead of hanging
            # what each flow may move in this tick: its demand, capped by its grant
            grants = [f.grant() for f in flows]
            demand = [sum(q[0] for q in queue), float("inf") if now <= dur else 0.0]
            room = [float("inf") if g["unlimited"] else max(0.0, g["granted_bytes"] - consumed[i]) for i, g in enumerate(grants)]
            want = [min(demand[i], room[i]) for i in range(2)]
            budget = cap * dt
            fair = budget / 2
            move = [min(want[0], fair), min(want[1], fair)]
            spare = budget - move[0] - move[1]
            for i in range(2):                       # max-min: what one flow leaves goes to the other
                extra = min(spare, want[i] - move[i])
                move[i] += extra
                spare -= extra
            left = move[0]
            while queue and left > 0:                # kv_transfer serves its requests in arrival order
                take = min(left, queue[0][0])
                queue[0][0] -= take
                left -= take
                if queue[0][0] <= 0:
                    done_ms.append((now - queue[0][1]) * 1e3)
                    queue.pop(0)
            consumed[0] += int(move[0])
            consumed[1] += int(move[1])
            kv.report(consumed[0], consumed[0], int(sum(q[0] for q in queue)))
            off.report(consumed[1], consumed[1], 1 << 40 if now <= dur else 0)
            if now - t_renew > 0.5:
                c.renew(kv)
                c.renew(off)
                t_renew = now
        elapsed = time.perf_counter() - t0
        c.unregister(kv)
        c.unregister(off)
    return {
        "policy": policy, "requests": len(arrivals), "unfinished": len(queue),
        "flow_time_p50_ms": ctl.percentile(done_ms, 0.5) if done_ms else float("nan"),
        "flow_time_p99_ms": ctl.percentile(done_ms, 0.99) if done_ms else float("nan"),
        "flow_time_mean_ms": sum(done_ms) / len(done_ms) if done_ms else float("nan"),
        "kv_transfer_gb": consumed[0] / 1e9, "offload_goodput_gbps": consumed[1] / 1e9 / min(elapsed, dur), "wall_s": elapsed,
    }


def run_processes(cfg: Config1 | None = None, policy: str = "target_track", msg: str = "8M") -> Dict[str, float]:
    """The experiment with the compatibility programs as the flows: `fabricd`, one `gpu_server link:<GB/s>` (a link that its
    clients share, first come first served) and two `cpu_client` processes that register themselves with the daemon
    (SKYGDR_DAEMON): kv_transfer as a Poisson request stream (SKYGDR_REQUESTS), kv_offload backlogged and stopped over its
    control port when the requests are through. Both keep two reads in flight so that the link never idles on a round trip.
    Flow times and rates are scraped from the clients' own summary lines."""
    import os
    import re
    import subprocess
    import time

    from . import FabricDaemon, send_control, wait_for_control
    from .. import build
    from .daemon import free_port

    cfg = cfg or Config1()
    bin_dir = str(build.build_bin())
    link_port, ctrl_port = free_port(), free_port()
    with FabricDaemon(policy=policy, window_us=int(cfg.window_ms * 1000), capacity_gbps=cfg.capacity_gbps, lease_ms=3000) as d:
        server = subprocess.Popen([f"{bin_dir}/gpu_server", f"link:{cfg.capacity_gbps}", "1G", str(link_port), "1", "0"], stdout=subprocess.PIPE, text=True)
        try:
            server.stdout.readline()                                            # "[server] ... listening"
            env = dict(os.environ, SKYGDR_DAEMON=f"127.0.0.1:{d.port}", SKYGDR_READ_MIN_QD="2")
            tail = ["read", "1", "0", "2"]                                      # op port gid_idx qd
            off_iters = int(cfg.capacity_gbps * 1e9 * (cfg.duration_s + 30) / (8 << 20))
            off = subprocess.Popen([f"{bin_dir}/cpu_client", "127.0.0.1", str(link_port), "link", str(off_iters), msg, *tail], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                   text=True, env=dict(env, SKYGDR_FLOW_NAME="kv_offload", SKYGDR_FLOW_PRIORITY="besteffort", SKYGDR_CTRL_PORT=str(ctrl_port)))
            wait_for_control("127.0.0.1", ctrl_port, 10.0)
            time.sleep(0.2)                                                     # the offload is up to speed before the requests start
            req = f"{cfg.rate_per_s}:{cfg.size_lo_mb * 1e6}:{cfg.size_hi_mb * 1e6}:{cfg.seed}:{cfg.duration_s}"
            kv = subprocess.run([f"{bin_dir}/cpu_client", "127.0.0.1", str(link_port), "link", "1", msg, *tail], capture_output=True, text=True, timeout=cfg.duration_s + 60,
                                env=dict(env, SKYGDR_FLOW_NAME="kv_transfer", SKYGDR_FLOW_PRIORITY="high", SKYGDR_FLOW_TARGET_GBPS=str(cfg.target_gbps), SKYGDR_REQUESTS=req))
            send_control("127.0.0.1", ctrl_port, "STOP")
            off_out, _ = off.communicate(timeout=30)
        finally:
            server.terminate()
            server.wait(timeout=5)
    m = re.search(r"requests=(\d+) finished=(\d+) unfinished=(\d+) flow_time_ms p50=([0-9.]+) p99=([0-9.]+) mean=([0-9.]+)", kv.stdout)
    if not m:
        raise RuntimeError("kv_transfer client gave no request summary:\n" + kv.stdout + kv.stderr)
    thr = re.search(r"throughput=([0-9.]+) GiB/s", off_out)
    return {"policy": policy, "requests": int(m.group(1)), "unfinished": int(m.group(3)), "flow_time_p50_ms": float(m.group(4)),
            "flow_time_p99_ms": float(m.group(5)), "flow_time_mean_ms": float(m.group(6)),
            "offload_goodput_gbps": float(thr.group(1)) * 1.073741824 if thr else float("nan")}


if __name__ == "__main__":
    import json
    import sys

    if "--processes" in sys.argv:
        print(json.dumps({p: run_processes(policy=p) for p in ("none", "target_track")}, indent=1))
    elif "--live" in sys.argv:
        print(json.dumps({p: run_live(policy=p) for p in ("none", "target_track")}, indent=1))
    else:
        print(json.dumps(run_config1(), indent=1))
