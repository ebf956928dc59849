"""Figures and tables of the PCIe contention study, redrawn from its two summary tables.

    python -m skygdr_b200.cli.contention_analyze --base_dir results/contention2_paper_v2

Same inputs, flag and figure names as the reference's script (src/tools/contention2_v2_analyze.py:806-880):

    <base_dir>/summary/partA_memcpy_impact.csv   one row per copy direction: the memcpy worker's bandwidth alone and next to
                                                 the network flow (mean / median / p95, sample counts, degradation_pct)
    <base_dir>/summary/partB_size_impact.csv     one row per message size: write and read throughput of the network flow
                                                 alone (`*_none_thr`) and next to a copy in the same direction
                                                 (`write_h2d_thr`, `read_d2h_thr`); ratios are computed when absent

The summaries are read as they are (hand edits are kept) and only the figures are redrawn, into <base_dir>/fig:

    partA_memcpy_impact_bar          bars: baseline vs contended copy bandwidth per direction, degradation on top
    partB_write_sweep_throughput     lines over message size: write alone (solid) vs +H2D (dashed)
    partB_read_sweep_throughput      the same for read vs +D2H
    partB_ratio_vs_size              contended / isolated throughput over message size, write and read
    partB_fourcases_throughput       the four cases of part B in one plot
    pcie_contention_combined         part A bars and part B ratios side by side

Every figure is written as `<name>.csv` (the numbers that are drawn) and `<name>.svg` (drawn here, no plotting library
needed), and also as `<name>.png` / `.pdf` when matplotlib can be imported. The raw-log readers the summaries are made
from are here too (`pcie_log_series`, `sweep_rows`, `gpu_metrics_active_util`), reading the `[pcie] t=...s ... bw_gib_s=...`
lines of gpu_pcie_memcpy, the CSV of msgsize_sweep and the CSV of gpu_metrics_logger; `--from_raw` builds both summaries
from a directory of such files named `partA_<dir>_{baseline,contended}.log` and `partB_{write,read}_{none,h2d,d2h}.csv`.
"""
from __future__ import annotations

import argparse
import csv
import math
import os
import re
import statistics
import sys
from typing import Dict, List, Optional, Sequence, Tuple

_PCIE_LINE = re.compile(r"t=([0-9.]+)s.*bw_gib_s=([0-9.]+)")
PALETTE = {"write": "#4C78A8", "read": "#F58518", "base": "#54A24B", "cont": "#E45756"}


# ---------------------------------------------------------------------------------------------------------------
# raw-log readers

def pcie_log_series(path: str) -> Dict[str, float]:
    """Bandwidth samples of a gpu_pcie_memcpy log -> n / mean / median / p95 (GiB/s)."""
    bw = [float(m.group(2)) for line in open(path) for m in [_PCIE_LINE.search(line)] if m]
    if not bw:
        return {"n": 0, "mean": float("nan"), "median": float("nan"), "p95": float("nan")}
    s = sorted(bw)
    return {"n": len(bw), "mean": statistics.fmean(bw), "median": statistics.median(bw), "p95": s[max(0, min(len(s) - 1, math.ceil(len(s) * 0.95) - 1))]}


def sweep_rows(path: str) -> Dict[int, Dict[str, float]]:
    """msgsize_sweep CSV -> {msg_bytes: {throughput_gib_s, p50_us, p99_us}} for the rows that ran (RetCode / rc 0)."""
    out = {}
    for row in csv.DictReader(open(path, newline="")):
        rc = row.get("RetCode", row.get("rc", "0")) or "0"
        if int(float(rc)) != 0:
            continue
        size = int(float(row.get("MsgBytes", row.get("msg_bytes"))))
        thr = float(row.get("Throughput_GiB_per_s", row.get("throughput_gib_s")))
        out[size] = {"throughput_gib_s": thr, "p50_us": _f(row.get("P50_us", row.get("p50_us"))), "p99_us": _f(row.get("P99_us", row.get("p99_us")))}
    return out


def gpu_metrics_active_util(path: str) -> Dict[str, float]:
    """gpu_metrics_logger CSV -> mean / p95 / peak of the busier PCIe direction over the samples that have a reading."""
    active = []
    for row in csv.DictReader(open(path, newline="")):
        tx, rx = _f(row.get("pcie_tx_util_pct")), _f(row.get("pcie_rx_util_pct"))
        vals = [v for v in (tx, rx) if not math.isnan(v) and v >= 0]
        if vals:
            active.append(max(vals))
    if not active:
        return {"n": 0, "mean": float("nan"), "p95": float("nan"), "peak": float("nan")}
    s = sorted(active)
    return {"n": len(s), "mean": statistics.fmean(s), "p95": s[max(0, min(len(s) - 1, math.ceil(len(s) * 0.95) - 1))], "peak": s[-1]}


def _f(v) -> float:
    try:
        return float(v)
    except (TypeError, ValueError):
        return float("nan")


# ---------------------------------------------------------------------------------------------------------------
# summaries

PART_A_COLS = ["direction", "baseline_mean_bw_gib_s", "baseline_median_bw_gib_s", "baseline_p95_bw_gib_s", "baseline_n",
               "contended_mean_bw_gib_s", "contended_median_bw_gib_s", "contended_p95_bw_gib_s", "contended_n", "degradation_pct"]
PART_B_COLS = ["msg_bytes", "write_none_thr", "write_h2d_thr", "read_none_thr", "read_d2h_thr", "write_thr_ratio", "read_thr_ratio"]


def load_part_a(path: str) -> List[Dict]:
    rows = []
    for r in csv.DictReader(open(path, newline="")):
        row = {"direction": r["direction"]}
        for c in PART_A_COLS[1:]:
            row[c] = _f(r.get(c))
        if math.isnan(row["degradation_pct"]) and row["baseline_mean_bw_gib_s"] > 0:
            row["degradation_pct"] = 100.0 * (1.0 - row["contended_mean_bw_gib_s"] / row["baseline_mean_bw_gib_s"])
        rows.append(row)
    return rows


def load_part_b(path: str) -> List[Dict]:
    rows = []
    for r in csv.DictReader(open(path, newline="")):
        missing = [c for c in PART_B_COLS[:5] if c not in r]
        if missing:
            raise ValueError(f"{path} misses the columns {missing}")
        row = {c: _f(r[c]) for c in PART_B_COLS[:5]}
        row["msg_bytes"] = int(row["msg_bytes"])
        for ratio, num, den in (("write_thr_ratio", "write_h2d_thr", "write_none_thr"), ("read_thr_ratio", "read_d2h_thr", "read_none_thr")):
            given = _f(r.get(ratio)) if r.get(ratio, "") != "" else float("nan")
            row[ratio] = given if not math.isnan(given) else (row[num] / row[den] if row[den] > 0 else float("nan"))
        rows.append(row)
    return sorted(rows, key=lambda x: x["msg_bytes"])


def summaries_from_raw(raw_dir: str, summary_dir: str) -> None:
    """Builds both summary tables from raw logs (see the module text for the file names); absent files leave rows out."""
    os.makedirs(summary_dir, exist_ok=True)
    a_rows = []
    for direction in ("h2d", "d2h"):
        b, c = os.path.join(raw_dir, f"partA_{direction}_baseline.log"), os.path.join(raw_dir, f"partA_{direction}_contended.log")
        if os.path.exists(b) and os.path.exists(c):
            sb, sc = pcie_log_series(b), pcie_log_series(c)
            deg = 100.0 * (1.0 - sc["mean"] / sb["mean"]) if sb["mean"] > 0 else float("nan")
            a_rows.append([direction, sb["mean"], sb["median"], sb["p95"], sb["n"], sc["mean"], sc["median"], sc["p95"], sc["n"], deg])
    if a_rows:
        _write_csv(os.path.join(summary_dir, "partA_memcpy_impact.csv"), PART_A_COLS, a_rows)
    names = {"write_none_thr": "partB_write_none.csv", "write_h2d_thr": "partB_write_h2d.csv", "read_none_thr": "partB_read_none.csv", "read_d2h_thr": "partB_read_d2h.csv"}
    cols = {k: sweep_rows(os.path.join(raw_dir, f)) for k, f in names.items() if os.path.exists(os.path.join(raw_dir, f))}
    if len(cols) == 4:
        sizes = sorted(set.intersection(*(set(v) for v in cols.values())))
        rows = []
        for s in sizes:
            v = {k: cols[k][s]["throughput_gib_s"] for k in names}
            rows.append([s, v["write_none_thr"], v["write_h2d_thr"], v["read_none_thr"], v["read_d2h_thr"],
                         v["write_h2d_thr"] / v["write_none_thr"] if v["write_none_thr"] > 0 else float("nan"),
                         v["read_d2h_thr"] / v["read_none_thr"] if v["read_none_thr"] > 0 else float("nan")])
        _write_csv(os.path.join(summary_dir, "partB_size_impact.csv"), PART_B_COLS, rows)


def _write_csv(path: str, header: Sequence[str], rows: Sequence[Sequence]) -> None:
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(header)
        w.writerows(rows)


# ---------------------------------------------------------------------------------------------------------------
# a small chart writer (SVG), so that the figures exist without a plotting library

def size_label(v: float) -> str:
    for unit, div in (("GiB", 1 << 30), ("MiB", 1 << 20), ("KiB", 1 << 10)):
        if v >= div:
            x = v / div
            return f"{x:.0f}{unit}" if abs(x - round(x)) < 1e-9 else f"{x:.1f}{unit}"
    return f"{int(v)}B"


class Svg:
    def __init__(self, w: int = 720, h: int = 420):
        self.w, self.h, self.parts = w, h, []

    def add(self, s: str) -> None:
        self.parts.append(s)

    def text(self, x, y, s, size=12, anchor="middle", rotate=None, color="#222"):
        tr = f' transform="rotate({rotate} {x:.1f} {y:.1f})"' if rotate is not None else ""
        self.add(f'<text x="{x:.1f}" y="{y:.1f}" font-size="{size}" text-anchor="{anchor}" fill="{color}" font-family="sans-serif"{tr}>{s}</text>')

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(f'<svg xmlns="http://www.w3.org/2000/svg" width="{self.w}" height="{self.h}" viewBox="0 0 {self.w} {self.h}">\n'
                    f'<rect width="{self.w}" height="{self.h}" fill="white"/>\n' + "\n".join(self.parts) + "\n</svg>\n")


def _axes(svg: Svg, box: Tuple[float, float, float, float], ymax: float, ylabel: str, title: str, yticks: int = 5) -> None:
    x0, y0, x1, y1 = box
    svg.add(f'<line x1="{x0}" y1="{y1}" x2="{x1}" y2="{y1}" stroke="#333"/><line x1="{x0}" y1="{y0}" x2="{x0}" y2="{y1}" stroke="#333"/>')
    for i in range(yticks + 1):
        v = ymax * i / yticks
        y = y1 - (y1 - y0) * i / yticks
        svg.add(f'<line x1="{x0}" y1="{y:.1f}" x2="{x1}" y2="{y:.1f}" stroke="#ddd"/>')
        svg.text(x0 - 6, y + 4, f"{v:.3g}", 11, "end")
    svg.text(x0 - 42, (y0 + y1) / 2, ylabel, 12, rotate=-90)
    svg.text((x0 + x1) / 2, y0 - 10, title, 13)


def bar_panel(svg: Svg, box, groups: Sequence[str], series: Sequence[Tuple[str, Sequence[float], str]], ylabel: str, title: str,
              notes: Optional[Sequence[str]] = None) -> None:
    """Grouped bars: `series` = (label, one value per group, colour); `notes` = a caption above every group."""
    x0, y0, x1, y1 = box
    ymax = max([v for _, vals, _ in series for v in vals if not math.isnan(v)] + [1e-9]) * 1.25
    _axes(svg, box, ymax, ylabel, title)
    gw = (x1 - x0) / max(1, len(groups))
    bw = gw * 0.7 / max(1, len(series))
    for gi, g in enumerate(groups):
        gx = x0 + gi * gw + gw * 0.15
        top = y1
        for si, (_, vals, color) in enumerate(series):
            v = vals[gi]
            if math.isnan(v):
                continue
            h = (y1 - y0) * v / ymax
            svg.add(f'<rect x="{gx + si * bw:.1f}" y="{y1 - h:.1f}" width="{bw * 0.92:.1f}" height="{h:.1f}" fill="{color}"/>')
            svg.text(gx + si * bw + bw * 0.46, y1 - h - 4, f"{v:.3g}", 10)
            top = min(top, y1 - h)
        svg.text(gx + gw * 0.35, y1 + 16, g, 12)
        if notes:
            svg.text(gx + gw * 0.35, top - 18, notes[gi], 11, color="#B22")
    for si, (label, _, color) in enumerate(series):
        svg.add(f'<rect x="{x1 - 150}" y="{y0 + 4 + si * 16}" width="10" height="10" fill="{color}"/>')
        svg.text(x1 - 136, y0 + 13 + si * 16, label, 11, "start")


def line_panel(svg: Svg, box, xs: Sequence[float], series: Sequence[Tuple[str, Sequence[float], str, bool]], ylabel: str, title: str,
               ymax: Optional[float] = None, hline: Optional[float] = None) -> None:
    """Lines over message size (log2 x axis): `series` = (label, values, colour, dashed)."""
    x0, y0, x1, y1 = box
    top = ymax or max([v for _, vals, _, _ in series for v in vals if not math.isnan(v)] + [1e-9]) * 1.15
    _axes(svg, box, top, ylabel, title)
    lx = [math.log2(max(1.0, x)) for x in xs]
    lo, hi = (min(lx), max(lx)) if lx else (0.0, 1.0)
    span = (hi - lo) or 1.0
    px = [x0 + (x1 - x0) * (0.04 + 0.92 * (v - lo) / span) for v in lx]
    step = max(1, len(xs) // 8)
    for i in range(0, len(xs), step):
        svg.text(px[i], y1 + 16, size_label(xs[i]), 10)
    if hline is not None:
        y = y1 - (y1 - y0) * hline / top
        svg.add(f'<line x1="{x0}" y1="{y:.1f}" x2="{x1}" y2="{y:.1f}" stroke="#999" stroke-dasharray="2 3"/>')
    for si, (label, vals, color, dashed) in enumerate(series):
        pts = [(px[i], y1 - (y1 - y0) * v / top) for i, v in enumerate(vals) if not math.isnan(v)]
        if pts:
            dash = ' stroke-dasharray="6 4"' if dashed else ""
            svg.add(f'<polyline fill="none" stroke="{color}" stroke-width="2"{dash} points="' + " ".join(f"{x:.1f},{y:.1f}" for x, y in pts) + '"/>')
            for x, y in pts:
                svg.add(f'<circle cx="{x:.1f}" cy="{y:.1f}" r="2.5" fill="{color}"/>')
        svg.add(f'<line x1="{x1 - 170}" y1="{y0 + 10 + si * 16}" x2="{x1 - 146}" y2="{y0 + 10 + si * 16}" stroke="{color}" stroke-width="2"'
                + (' stroke-dasharray="6 4"' if dashed else "") + "/>")
        svg.text(x1 - 140, y0 + 14 + si * 16, label, 11, "start")
    svg.text((x0 + x1) / 2, y1 + 34, "message size", 12)


def _maybe_matplotlib(name: str, fig_dir: str, draw) -> None:
    """The same figure through matplotlib (PNG and PDF) where it is installed; silently nothing where it is not."""
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        return
    fig = draw(plt)
    fig.tight_layout()
    fig.savefig(os.path.join(fig_dir, name + ".png"), dpi=150)
    fig.savefig(os.path.join(fig_dir, name + ".pdf"))
    plt.close(fig)


# ---------------------------------------------------------------------------------------------------------------
# the figures

def fig_part_a(rows: List[Dict], fig_dir: str) -> None:
    name = "partA_memcpy_impact_bar"
    groups = [r["direction"].upper() for r in rows]
    base, cont = [r["baseline_mean_bw_gib_s"] for r in rows], [r["contended_mean_bw_gib_s"] for r in rows]
    notes = [f"-{r['degradation_pct']:.1f}%" for r in rows]
    _write_csv(os.path.join(fig_dir, name + ".csv"), ["direction", "baseline_mean_bw_gib_s", "contended_mean_bw_gib_s", "degradation_pct"],
               [[r["direction"], r["baseline_mean_bw_gib_s"], r["contended_mean_bw_gib_s"], r["degradation_pct"]] for r in rows])
    svg = Svg()
    bar_panel(svg, (80, 50, 690, 360), groups, [("copy alone", base, PALETTE["base"]), ("copy next to the network flow", cont, PALETTE["cont"])],
              "copy bandwidth (GiB/s)", "Part A: what the network flow costs the memcpy worker", notes)
    svg.save(os.path.join(fig_dir, name + ".svg"))

    def draw(plt):
        fig, ax = plt.subplots(figsize=(6, 4))
        x = range(len(groups))
        ax.bar([i - 0.2 for i in x], base, 0.4, label="copy alone", color=PALETTE["base"])
        ax.bar([i + 0.2 for i in x], cont, 0.4, label="next to the network flow", color=PALETTE["cont"])
        ax.set_xticks(list(x)); ax.set_xticklabels(groups); ax.set_ylabel("copy bandwidth (GiB/s)"); ax.legend()
        return fig

    _maybe_matplotlib(name, fig_dir, draw)


def fig_part_b_sweep(rows: List[Dict], fig_dir: str, op: str) -> None:
    none_col, cont_col, cont_name = (("write_none_thr", "write_h2d_thr", "+H2D") if op == "write" else ("read_none_thr", "read_d2h_thr", "+D2H"))
    name = f"partB_{op}_sweep_throughput"
    xs = [r["msg_bytes"] for r in rows]
    _write_csv(os.path.join(fig_dir, name + ".csv"), ["msg_bytes", "isolated_gib_s", "contended_gib_s"], [[r["msg_bytes"], r[none_col], r[cont_col]] for r in rows])
    svg = Svg()
    line_panel(svg, (80, 50, 690, 350), xs, [(f"{op} alone", [r[none_col] for r in rows], PALETTE[op], False),
                                             (f"{op} {cont_name}", [r[cont_col] for r in rows], PALETTE[op], True)],
               "throughput (GiB/s)", f"Part B {op} sweep: isolated vs {cont_name}")
    svg.save(os.path.join(fig_dir, name + ".svg"))

    def draw(plt):
        fig, ax = plt.subplots(figsize=(6.5, 4))
        ax.plot(xs, [r[none_col] for r in rows], "-o", color=PALETTE[op], label=f"{op} alone")
        ax.plot(xs, [r[cont_col] for r in rows], "--o", color=PALETTE[op], label=f"{op} {cont_name}")
        ax.set_xscale("log", base=2); ax.set_xlabel("message size (bytes)"); ax.set_ylabel("throughput (GiB/s)"); ax.legend()
        return fig

    _maybe_matplotlib(name, fig_dir, draw)


def fig_part_b_ratio(rows: List[Dict], fig_dir: str) -> None:
    name = "partB_ratio_vs_size"
    xs = [r["msg_bytes"] for r in rows]
    _write_csv(os.path.join(fig_dir, name + ".csv"), ["msg_bytes", "write_thr_ratio", "read_thr_ratio"], [[r["msg_bytes"], r["write_thr_ratio"], r["read_thr_ratio"]] for r in rows])
    svg = Svg()
    line_panel(svg, (80, 50, 690, 350), xs, [("write +H2D / write alone", [r["write_thr_ratio"] for r in rows], PALETTE["write"], False),
                                             ("read +D2H / read alone", [r["read_thr_ratio"] for r in rows], PALETTE["read"], False)],
               "contended / isolated throughput", "Part B: share of the isolated throughput kept under contention", ymax=1.2, hline=1.0)
    svg.save(os.path.join(fig_dir, name + ".svg"))

    def draw(plt):
        fig, ax = plt.subplots(figsize=(6.5, 4))
        ax.plot(xs, [r["write_thr_ratio"] for r in rows], "-o", color=PALETTE["write"], label="write +H2D / alone")
        ax.plot(xs, [r["read_thr_ratio"] for r in rows], "-o", color=PALETTE["read"], label="read +D2H / alone")
        ax.axhline(1.0, color="#999", linestyle=":"); ax.set_xscale("log", base=2); ax.set_ylim(0, 1.2); ax.legend()
        return fig

    _maybe_matplotlib(name, fig_dir, draw)


def fig_part_b_four(rows: List[Dict], fig_dir: str) -> None:
    name = "partB_fourcases_throughput"
    xs = [r["msg_bytes"] for r in rows]
    cases = [("write alone", "write_none_thr", PALETTE["write"], False), ("write +H2D", "write_h2d_thr", PALETTE["write"], True),
             ("read alone", "read_none_thr", PALETTE["read"], False), ("read +D2H", "read_d2h_thr", PALETTE["read"], True)]
    _write_csv(os.path.join(fig_dir, name + ".csv"), ["msg_bytes"] + [c[1] for c in cases], [[r["msg_bytes"]] + [r[c[1]] for c in cases] for r in rows])
    svg = Svg()
    line_panel(svg, (80, 50, 690, 350), xs, [(label, [r[col] for r in rows], color, dashed) for label, col, color, dashed in cases],
               "throughput (GiB/s)", "Part B: the four cases")
    svg.save(os.path.join(fig_dir, name + ".svg"))

    def draw(plt):
        fig, ax = plt.subplots(figsize=(6.5, 4))
        for label, col, color, dashed in cases:
            ax.plot(xs, [r[col] for r in rows], "--o" if dashed else "-o", color=color, label=label)
        ax.set_xscale("log", base=2); ax.set_xlabel("message size (bytes)"); ax.set_ylabel("throughput (GiB/s)"); ax.legend()
        return fig

    _maybe_matplotlib(name, fig_dir, draw)


def fig_combined(a_rows: List[Dict], b_rows: List[Dict], fig_dir: str) -> None:
    name = "pcie_contention_combined"
    svg = Svg(1180, 430)
    bar_panel(svg, (80, 55, 540, 360), [r["direction"].upper() for r in a_rows],
              [("copy alone", [r["baseline_mean_bw_gib_s"] for r in a_rows], PALETTE["base"]),
               ("copy next to the network flow", [r["contended_mean_bw_gib_s"] for r in a_rows], PALETTE["cont"])],
              "copy bandwidth (GiB/s)", "(a) memcpy worker", [f"-{r['degradation_pct']:.1f}%" for r in a_rows])
    xs = [r["msg_bytes"] for r in b_rows]
    line_panel(svg, (680, 55, 1150, 350), xs, [("write +H2D / alone", [r["write_thr_ratio"] for r in b_rows], PALETTE["write"], False),
                                               ("read +D2H / alone", [r["read_thr_ratio"] for r in b_rows], PALETTE["read"], False)],
               "contended / isolated", "(b) network flow", ymax=1.2, hline=1.0)
    svg.save(os.path.join(fig_dir, name + ".svg"))
    _write_csv(os.path.join(fig_dir, name + ".csv"), ["panel", "x", "series", "value"],
               [["a", r["direction"], "baseline", r["baseline_mean_bw_gib_s"]] for r in a_rows] +
               [["a", r["direction"], "contended", r["contended_mean_bw_gib_s"]] for r in a_rows] +
               [["b", r["msg_bytes"], "write_ratio", r["write_thr_ratio"]] for r in b_rows] +
               [["b", r["msg_bytes"], "read_ratio", r["read_thr_ratio"]] for r in b_rows])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base_dir", default="results/contention2_paper_v2")
    ap.add_argument("--from_raw", default="", help="directory of raw logs to build the two summary tables from first")
    a = ap.parse_args(argv)
    fig_dir, summary_dir = os.path.join(a.base_dir, "fig"), os.path.join(a.base_dir, "summary")
    os.makedirs(fig_dir, exist_ok=True)
    if a.from_raw:
        summaries_from_raw(a.from_raw, summary_dir)
    part_a_csv, part_b_csv = os.path.join(summary_dir, "partA_memcpy_impact.csv"), os.path.join(summary_dir, "partB_size_impact.csv")
    if not os.path.exists(part_b_csv):
        print(f"missing summary csv: {part_b_csv}", file=sys.stderr)
        return 1
    b_rows = load_part_b(part_b_csv)
    if os.path.exists(part_a_csv):
        a_rows = load_part_a(part_a_csv)
        fig_part_a(a_rows, fig_dir)
        fig_combined(a_rows, b_rows, fig_dir)
    else:
        print(f"[warn] skip Part A plot; summary not found: {part_a_csv}")
    fig_part_b_sweep(b_rows, fig_dir, "write")
    fig_part_b_sweep(b_rows, fig_dir, "read")
    fig_part_b_ratio(b_rows, fig_dir)
    fig_part_b_four(b_rows, fig_dir)
    print(f"[ok] summary (read-only): {summary_dir}")
    print(f"[ok] fig: {fig_dir}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
