"""Runs the PCIe copy task and the HBM utilisation logger side by side and joins their samples.

    python -m skygdr_b200.cli.run_pcie_memcpy_with_bandwidth --out merged.csv [--bw_interval_ms 100] -- <gpu_pcie_memcpy flags>

Same job as src/tools/run_pcie_memcpy_with_bandwidth.py: scrape the `[pcie]` lines (regex of :23-27), sample memory
utilisation, and as-of join every `[pcie]` row with the latest bandwidth sample (:229-306).
"""
from __future__ import annotations

import argparse
import bisect
import csv
import re
import subprocess
import sys
import time

PCIE_RE = re.compile(r"\[pcie\]\s+t=([0-9.]+)s\s+dir=(\w+)\s+bw_gib_s=([0-9.]+)\s+bytes=(\d+)")


def parse_pcie_lines(text: str):
    return [{"t_s": float(m.group(1)), "dir": m.group(2), "bw_gib_s": float(m.group(3)), "bytes": int(m.group(4))} for m in PCIE_RE.finditer(text)]


def asof_join(pcie_rows, bw_rows):
    """Each pcie row gets the last bandwidth sample at or before its time."""
    ts = [b["t_s"] for b in bw_rows]
    out = []
    for r in pcie_rows:
        i = bisect.bisect_right(ts, r["t_s"]) - 1
        b = bw_rows[i] if i >= 0 else {}
        out.append({**r, "memory_util_pct": b.get("memory_util_pct", ""), "estimated_mem_bw_GB_s": b.get("estimated_mem_bw_GB_s", "")})
    return out


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    extra = []
    if "--" in argv:
        i = argv.index("--")
        argv, extra = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--bw_interval_ms", type=int, default=100)
    a = ap.parse_args(argv)
    from skygdr_b200.control import ctl

    sig = ctl.GpuSignals(a.gpu)
    proc = subprocess.Popen([sys.executable, "-m", "skygdr_b200.cli.gpu_pcie_memcpy", *extra], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    t0 = time.time()
    bw_rows = []
    while proc.poll() is None:
        if sig.available:
            s = sig.sample_hbm()
            bw_rows.append({"t_s": time.time() - t0, "memory_util_pct": s.memory_util_pct, "estimated_mem_bw_GB_s": s.estimated_gb_s})
        time.sleep(max(a.bw_interval_ms, 50) / 1000.0)
    text = proc.stdout.read()
    rows = asof_join(parse_pcie_lines(text), bw_rows)
    with open(a.out, "w", newline="") as fp:
        w = csv.DictWriter(fp, fieldnames=["t_s", "dir", "bw_gib_s", "bytes", "memory_util_pct", "estimated_mem_bw_GB_s"])
        w.writeheader()
        w.writerows(rows)
    print(f"merged {len(rows)} rows -> {a.out}")
    return proc.returncode or 0


if __name__ == "__main__":
    raise SystemExit(main())
