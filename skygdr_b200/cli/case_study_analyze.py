"""Joins a controller CSV with the background flow's time series and summarises a case-study run.

    python -m skygdr_b200.cli.case_study_analyze --controller_csv C.csv --bg_ts_csv T.csv --out_csv merged.csv [--out_png P.png]
           [--always_high_restore_csv A.csv --always_low_restore_csv B.csv --controlled_restore_csv C.csv]

Follows src/tools/pcie_case_study_analyze.py: the two files may come from hosts whose clocks differ, so the offset
is estimated by matching the sequence of mode changes seen by both (:103-137); every controller row then gets the
background sample nearest in time (:197-247); the summary prints restore_finish_ms, low_samples and
bg_throughput_mean_gib_s (:505-515). The three optional restore CSVs are the arms of the study (no scheduling,
static throttle, controlled) and are reduced to their finish times. Plots need matplotlib and are optional.
"""
from __future__ import annotations

import argparse
import csv
import sys
from typing import Dict, List, Optional


def read_csv(path: str) -> List[Dict[str, str]]:
    with open(path) as f:
        return list(csv.DictReader(f))


def mode_transitions(rows: List[Dict[str, str]], mode_key: str, ts_key: str = "ts_unix_ms"):
    out, prev = [], None
    for r in rows:
        m = r.get(mode_key, "")
        if m != prev and m:
            out.append((m, float(r[ts_key])))
            prev = m
    return out


def estimate_clock_offset_ms(ctrl_rows, bg_rows) -> float:
    """Median of (bg time - controller time) over mode changes that appear in the same order in both files."""
    a = mode_transitions(ctrl_rows, "mode")
    b = mode_transitions(bg_rows, "control_mode")
    diffs, j = [], 0
    for m, t in a[1:]:                       # the initial mode is not a change: both sides start in it at unrelated times
        k = j
        while k < len(b) and b[k][0] != m:
            k += 1
        if k < len(b):                       # a mode the coarser file never shows is skipped, not allowed to derail the rest
            diffs.append(b[k][1] - t)
            j = k + 1
    if not diffs:
        return 0.0
    diffs.sort()
    return diffs[len(diffs) // 2]


def merge(ctrl_rows, bg_rows, offset_ms: float):
    bg_t = [float(r["ts_unix_ms"]) - offset_ms for r in bg_rows]
    out, j = [], 0
    for r in ctrl_rows:
        t = float(r["ts_unix_ms"])
        while j + 1 < len(bg_t) and abs(bg_t[j + 1] - t) <= abs(bg_t[j] - t):
            j += 1
        b = bg_rows[j] if bg_rows else {}
        out.append({**r, "bg_throughput_gib_s": b.get("throughput_gib_s", ""), "bg_p99_us": b.get("p99_us", ""),
                    "bg_control_mode": b.get("control_mode", ""), "bg_pace_sleep_us": b.get("pace_sleep_us", "")})
    return out


def restore_finish_ms(rows: List[Dict[str, str]]) -> Optional[float]:
    for r in rows:
        if r.get("done", r.get("restore_done", "0")) in ("1", "1.0"):
            return float(r.get("elapsed_ms", r.get("restore_elapsed_ms", "nan")))
    return None


def summarise(merged) -> Dict[str, float]:
    low = [r for r in merged if r["mode"].startswith("LOW") or r["mode"].startswith("SLEEP")]
    bg = [float(r["bg_throughput_gib_s"]) for r in merged if r["bg_throughput_gib_s"] not in ("", None)]
    fin = restore_finish_ms(merged)
    return {"restore_finish_ms": fin if fin is not None else float("nan"), "low_samples": len(low),
            "bg_throughput_mean_gib_s": sum(bg) / len(bg) if bg else float("nan")}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--controller_csv", required=True)
    ap.add_argument("--bg_ts_csv", required=True)
    ap.add_argument("--out_csv", required=True)
    ap.add_argument("--out_png", default="")
    ap.add_argument("--paper_out_pdf", default="")
    ap.add_argument("--plot_start_s", type=float, default=0.0)
    ap.add_argument("--plot_end_s", type=float, default=0.0)
    ap.add_argument("--rx_threshold_pct", type=float, default=85.0)
    ap.add_argument("--pcie_peak_gib_s", type=float, default=29.0)
    ap.add_argument("--always_high_restore_csv", default="")
    ap.add_argument("--always_low_restore_csv", default="")
    ap.add_argument("--controlled_restore_csv", default="")
    a = ap.parse_args(argv)
    ctrl, bg = read_csv(a.controller_csv), read_csv(a.bg_ts_csv)
    off = estimate_clock_offset_ms(ctrl, bg)
    merged = merge(ctrl, bg, off)
    if merged:
        with open(a.out_csv, "w", newline="") as fp:
            w = csv.DictWriter(fp, fieldnames=list(merged[0].keys()))
            w.writeheader()
            w.writerows(merged)
    s = summarise(merged)
    print(f"clock_offset_ms={off:.1f}")
    for k, v in s.items():
        print(f"{k}={v}")
    for name in ("always_high", "always_low", "controlled"):
        p = getattr(a, f"{name}_restore_csv")
        if p:
            print(f"{name}_restore_finish_ms={restore_finish_ms(read_csv(p))}")
    if a.out_png or a.paper_out_pdf:
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt

            t0 = float(merged[0]["ts_unix_ms"])
            t = [(float(r["ts_unix_ms"]) - t0) / 1e3 for r in merged]
            fig, ax = plt.subplots(2, 1, figsize=(9, 6), sharex=True)
            ax[0].plot(t, [float(r["restore_guard_bw_gib_s"] or "nan") for r in merged], label="protected (H2D)")
            ax[0].plot(t, [float(r["bg_throughput_gib_s"] or "nan") for r in merged], label="background")
            ax[0].axhline(a.pcie_peak_gib_s, ls=":", c="gray"); ax[0].set_ylabel("GiB/s"); ax[0].legend()
            ax[1].plot(t, [float(r["pcie_rx_util_pct"] or "nan") for r in merged]); ax[1].axhline(a.rx_threshold_pct, ls=":", c="r")
            ax[1].set_ylabel("PCIe RX util %"); ax[1].set_xlabel("s")
            for out in (a.out_png, a.paper_out_pdf):
                if out:
                    fig.savefig(out, dpi=120)
        except Exception as exc:
            print(f"plot skipped: {exc}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
