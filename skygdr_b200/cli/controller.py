"""The signal -> policy -> action loop of the PCIe case study, as a command-line program.

    python -m skygdr_b200.cli.controller --cpu_control_host H --cpu_control_port P --baseline_restore_gib_s B --log_dir D
        [--policy ladder|target_track|weighted_track] [--poll_ms 100] [--restore_total_bytes 64G] [--restore_max_outstanding_bytes 4G] ...

Arguments, output files (`<tag>_{restore_progress,gpu_metrics,controller}.csv`), the 18-column controller CSV and
the decision names (HOLD | SWITCH_LOW1 | ESCALATE_LOWn | RESTORE_DONE_HIGH | STOP) are those of
src/tools/pcie_case_study_controller.py:134-171,179-183,250-271,290-320. The protected flow is the local restore
(gpu_pcie_memcpy, finite --total_bytes); the background flow is a remote end-point reached through its control
port. Differences: the decision rule is this runtime's C++ policy object (`ladder` reproduces the reference rule,
`target_track` also uses exit_ratio/exit_windows, which the reference parses but never applies); the poll period
may go down to 5 ms; a stale-sample guard rejects rows older than the run (reference :71-79).
"""
from __future__ import annotations

import argparse
import csv
import math
import os
import subprocess
import sys
import time
from typing import Dict, Optional

from .common import parse_size


def read_last_csv_row(path: str) -> Optional[Dict[str, str]]:
    """Last complete row of a CSV that another process is appending to."""
    try:
        with open(path, "rb") as f:
            f.seek(0, os.SEEK_END)
            size = f.tell()
            f.seek(0)
            head = f.readline().decode(errors="replace").strip()
            if not head:
                return None
            f.seek(max(0, size - 4096))
            tail = f.read().decode(errors="replace")
    except OSError:
        return None
    lines = [l for l in tail.splitlines() if l.strip()]
    if not tail.endswith("\n") and lines:
        lines = lines[:-1]                       # a half-written last line
    cols = head.split(",")
    for line in reversed(lines):
        vals = line.split(",")
        if len(vals) == len(cols) and vals != cols:
            return dict(zip(cols, vals))
    return None


def fresh_row(row: Optional[Dict[str, str]], run_start_unix_ms: int) -> Optional[Dict[str, str]]:
    """Rejects a row written before this run started (a file left over from an earlier run)."""
    if not row:
        return None
    try:
        return row if int(float(row.get("ts_unix_ms", "0"))) >= run_start_unix_ms else None
    except ValueError:
        return None


def to_float(v) -> float:
    try:
        return float(v)
    except (TypeError, ValueError):
        return float("nan")


def terminate(proc: Optional[subprocess.Popen]) -> None:
    if proc is None or proc.poll() is not None:
        return
    try:
        proc.terminate()
        proc.wait(timeout=3)
    except Exception:
        try:
            proc.kill()
            proc.wait(timeout=2)
        except Exception:
            print("[warn] child did not stop cleanly", file=sys.stderr)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu_control_host", required=True)
    ap.add_argument("--cpu_control_port", type=int, required=True)
    ap.add_argument("--control_timeout_s", type=float, default=15.0)
    ap.add_argument("--python_bin", default=sys.executable)
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--gpu_metrics_interval_ms", type=int, default=100)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--dir", default="h2d")
    ap.add_argument("--chunk_mb", type=int, default=128)
    ap.add_argument("--streams", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--inflight", type=int, default=4)
    ap.add_argument("--pinned", type=int, default=1)
    ap.add_argument("--baseline_restore_gib_s", type=float, required=True)
    ap.add_argument("--restore_total_bytes", default="64G")
    ap.add_argument("--restore_max_outstanding_bytes", default="4G")
    ap.add_argument("--progress_ms", type=int, default=100)
    ap.add_argument("--progress_smooth_windows", type=int, default=5)
    ap.add_argument("--poll_ms", type=int, default=100)
    ap.add_argument("--warmup_ms", type=int, default=1000)
    ap.add_argument("--post_restore_ms", type=int, default=2000)
    ap.add_argument("--enter_ratio", type=float, default=0.65)
    ap.add_argument("--exit_ratio", type=float, default=0.80)
    ap.add_argument("--rx_threshold_pct", type=float, default=85.0)
    ap.add_argument("--enter_windows", type=int, default=1)
    ap.add_argument("--exit_windows", type=int, default=2)
    ap.add_argument("--log_dir", required=True)
    ap.add_argument("--tag", default="case_study")
    ap.add_argument("--policy", default="ladder", choices=["ladder", "target_track", "weighted_track", "none", "static"])
    ap.add_argument("--pcie_bin", default="", help="program of the protected flow (reference flag); default: this package's gpu_pcie_memcpy")
    ap.add_argument("--gpu_metrics_script", default="", help="signal logger script (reference flag); default: this package's gpu_metrics_logger")
    ap.add_argument("--restore_cmd", default="", help="override the protected-flow command (must write the progress CSV given by {progress})")
    ap.add_argument("--metrics_cmd", default="", help="override the signal command (must write the metrics CSV given by {metrics})")
    ap.add_argument("--min_poll_ms", type=int, default=5)
    return ap


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    from skygdr_b200.control import ctl, send_control, wait_for_control

    os.makedirs(a.log_dir, exist_ok=True)
    progress_csv = os.path.join(a.log_dir, f"{a.tag}_restore_progress.csv")
    metrics_csv = os.path.join(a.log_dir, f"{a.tag}_gpu_metrics.csv")
    controller_csv = os.path.join(a.log_dir, f"{a.tag}_controller.csv")
    baseline = a.baseline_restore_gib_s
    enter_thresh, exit_thresh = baseline * a.enter_ratio, baseline * a.exit_ratio
    total_bytes = parse_size(a.restore_total_bytes)
    pc = ctl.PolicyConfig()
    pc.enter_ratio, pc.exit_ratio, pc.util_threshold_pct = a.enter_ratio, a.exit_ratio, a.rx_threshold_pct
    pc.enter_windows, pc.exit_windows = a.enter_windows, a.exit_windows
    policy = ctl.make_policy(a.policy, pc)
    try:
        wait_for_control(a.cpu_control_host, a.cpu_control_port, a.control_timeout_s)
    except RuntimeError as exc:
        print(f"[controller] {exc}", file=sys.stderr)
        return 2
    response = send_control(a.cpu_control_host, a.cpu_control_port, "HIGH")
    run_start = int(time.time() * 1000)
    metrics_head = [a.python_bin, a.gpu_metrics_script] if a.gpu_metrics_script else [a.python_bin, "-m", "skygdr_b200.cli.gpu_metrics_logger"]
    restore_head = [a.pcie_bin] if a.pcie_bin else [a.python_bin, "-m", "skygdr_b200.cli.gpu_pcie_memcpy"]
    metrics_cmd = (a.metrics_cmd.format(metrics=metrics_csv).split() if a.metrics_cmd else
                   [*metrics_head, "--gpu", str(a.gpu), "--interval_ms",
                    str(a.gpu_metrics_interval_ms), "--out", metrics_csv])
    restore_cmd = (a.restore_cmd.format(progress=progress_csv).split() if a.restore_cmd else
                   [*restore_head, f"--device={a.device}", "--seconds=0", f"--dir={a.dir}",
                    f"--chunk_mb={a.chunk_mb}", f"--streams={a.streams}", f"--batch={a.batch}", f"--inflight={a.inflight}",
                    f"--pinned={a.pinned}", f"--total_bytes={total_bytes}", f"--max_outstanding_bytes={a.restore_max_outstanding_bytes}",
                    f"--progress_ms={a.progress_ms}", f"--progress_smooth_windows={a.progress_smooth_windows}",
                    f"--progress_out={progress_csv}", f"--report_ms={max(a.progress_ms, 1000)}"])
    metrics_proc = restore_proc = None
    mode, stop_sent, deadline = "HIGH", False, None
    rc = 0
    try:
        metrics_proc = subprocess.Popen(metrics_cmd, stdout=open(os.path.join(a.log_dir, f"{a.tag}_gpu_metrics.log"), "w"), stderr=subprocess.STDOUT)
        time.sleep(max(a.warmup_ms, 0) / 1000.0)
        restore_proc = subprocess.Popen(restore_cmd, stdout=open(os.path.join(a.log_dir, f"{a.tag}_restore.log"), "w"), stderr=subprocess.STDOUT)
        with open(controller_csv, "w", newline="") as fp:
            w = csv.writer(fp)
            w.writerow(["ts_unix_ms", "mode", "decision", "restore_done", "restore_elapsed_ms", "restore_issued_bytes",
                        "restore_completed_bytes", "restore_remaining_bytes", "restore_inst_bw_gib_s", "restore_smooth_bw_gib_s",
                        "restore_guard_bw_gib_s", "restore_avg_bw_gib_s", "pcie_tx_util_pct", "pcie_rx_util_pct",
                        "baseline_restore_gib_s", "enter_thresh_gib_s", "exit_thresh_gib_s", "control_response"])
            while True:
                now_ms = int(time.time() * 1000)
                row = fresh_row(read_last_csv_row(progress_csv), run_start)
                mrow = fresh_row(read_last_csv_row(metrics_csv), run_start)
                g = lambda k, d=0: int(float(row.get(k, d))) if row else d
                inst, smooth, avg = (to_float(row.get(k)) if row else float("nan") for k in ("inst_bw_gib_s", "smooth_bw_gib_s", "avg_bw_gib_s"))
                guard = smooth if not math.isnan(smooth) else inst
                remaining = g("remaining_bytes", total_bytes)
                tx = to_float(mrow.get("pcie_tx_util_pct")) if mrow else float("nan")
                rx = to_float(mrow.get("pcie_rx_util_pct")) if mrow else float("nan")
                decision, response, done = "HOLD", "", False
                if row:
                    done = bool(g("done")) or remaining <= 0
                    if done:
                        inst = smooth = guard = 0.0
                    if not done:
                        s = ctl.FlowSignal()
                        s.id, s.priority, s.target_gbps = 1, 100, baseline       # the policy compares in the units it is given
                        s.inst_gbps, s.smooth_gbps, s.backlog_bytes, s.active = inst, guard, max(remaining, 1), True
                        bg = ctl.FlowSignal()
                        bg.id, bg.priority, bg.target_gbps, bg.backlog_bytes, bg.active = 2, 0, 0.0, 1, True
                        link = ctl.LinkSignal()
                        link.capacity_gbps, link.util_pct = max(baseline, 1e-9), rx
                        d = policy.step([s, bg], link)[1]
                        target = ctl.mode_name(d.mode) if d.mode != 6 else f"SLEEP {int(max(0.0, (1.0 / max(d.budget_gbps / baseline, 1e-3) - 1.0)) * 100)}"
                        if target != mode:
                            response = send_control(a.cpu_control_host, a.cpu_control_port, target)
                            decision = d.decision if d.decision != "HOLD" else f"SWITCH_{target.split()[0]}"
                            mode = target
                    elif deadline is None:
                        response = send_control(a.cpu_control_host, a.cpu_control_port, "HIGH")
                        mode, decision = "HIGH", "RESTORE_DONE_HIGH"
                        deadline = now_ms + max(a.post_restore_ms, 0)
                        policy.reset()
                    elif not stop_sent and now_ms >= deadline:
                        response = send_control(a.cpu_control_host, a.cpu_control_port, "STOP")
                        mode, decision, stop_sent = "STOP", "STOP", True
                f6 = lambda v: "" if math.isnan(v) else f"{v:.6f}"
                w.writerow([now_ms, mode, decision, 1 if done else 0, g("elapsed_ms"), g("issued_bytes"), g("completed_bytes"), remaining,
                            f6(inst), f6(smooth), f6(guard), f6(avg), f6(tx), f6(rx), f"{baseline:.6f}", f"{enter_thresh:.6f}",
                            f"{exit_thresh:.6f}", response])
                fp.flush()
                exited = restore_proc.poll() is not None
                if stop_sent and exited:
                    break
                if exited and deadline is None:
                    # The protected flow has exited and this pass did not see it finish. Its last row may have been written
                    # just before it exited, after this pass read the file: read once more. If it still is not done, the
                    # flow died on the way (reference: the loop ends whenever the restore process exits before RESTORE_DONE,
                    # src/tools/pcie_case_study_controller.py:349); the background flow is not left in a LOW mode.
                    last = fresh_row(read_last_csv_row(progress_csv), run_start)
                    finished = bool(last) and (int(float(last.get("done", 0))) != 0 or int(float(last.get("remaining_bytes", 1))) <= 0)
                    if not finished:
                        for cmd in ("HIGH", "STOP"):
                            try:
                                response = send_control(a.cpu_control_host, a.cpu_control_port, cmd)
                            except OSError:
                                break
                        w.writerow([int(time.time() * 1000), "STOP", "RESTORE_DIED_STOP", 0, g("elapsed_ms"), g("issued_bytes"), g("completed_bytes"),
                                    remaining, "", "", "", "", "", "", f"{baseline:.6f}", f"{enter_thresh:.6f}", f"{exit_thresh:.6f}", response])
                        fp.flush()
                        rc = 3
                        break
                time.sleep(max(a.poll_ms, a.min_poll_ms) / 1000.0)
    except KeyboardInterrupt:
        try:
            send_control(a.cpu_control_host, a.cpu_control_port, "STOP")
        except OSError:
            pass
        rc = 130
    finally:
        terminate(restore_proc)
        terminate(metrics_proc)
    return rc


if __name__ == "__main__":
    raise SystemExit(main())
