"""PCIe TX/RX (and optionally NVLink, HBM) signal logger.

    python -m skygdr_b200.cli.gpu_metrics_logger --gpu 0 --interval_ms 200 --out - [--append] [--live] [--duration_s 0]
                                                 [--nvlink] [--plot --plot_in CSV --plot_out PNG --plot_title T]

CSV columns and the utilisation rule (throughput over the MAX link generation x width) are those of
src/tools/gpu_metrics_logger.py:38-67,298-303. With --nvlink two more columns follow (nvlink_tx_GB_s, nvlink_rx_GB_s).
Sampling is native (skygdr_b200/csrc/ctl/signals.hpp); plotting needs matplotlib and is optional.
"""
from __future__ import annotations

import argparse
import os
import sys
import time


def plot(csv_in: str, png_out: str, title: str) -> int:
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception as exc:
        print(f"plot skipped: {exc}", file=sys.stderr)
        return 1
    import csv

    rows = list(csv.DictReader(open(csv_in)))
    t = [float(r["t_ms"]) / 1e3 for r in rows]
    fig, ax = plt.subplots(3, 1, figsize=(9, 8), sharex=True)
    ax[0].plot(t, [float(r["pcie_tx_GiB_s"]) for r in rows], label="TX")
    ax[0].plot(t, [float(r["pcie_rx_GiB_s"]) for r in rows], label="RX")
    ax[0].set_ylabel("GiB/s"); ax[0].legend()
    ax[1].plot(t, [float(r["pcie_tx_util_pct"]) for r in rows]); ax[1].set_ylabel("TX util %")
    ax[2].plot(t, [float(r["pcie_rx_util_pct"]) for r in rows]); ax[2].set_ylabel("RX util %"); ax[2].set_xlabel("s")
    fig.suptitle(title)
    fig.savefig(png_out, dpi=120)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--interval_ms", type=int, default=200)
    ap.add_argument("--out", default="-")
    ap.add_argument("--append", action="store_true")
    ap.add_argument("--live", action="store_true")
    ap.add_argument("--duration_s", type=float, default=0.0)
    ap.add_argument("--nvlink", action="store_true")
    ap.add_argument("--plot", action="store_true")
    ap.add_argument("--plot_in", default="")
    ap.add_argument("--plot_out", default="gpu_metrics.png")
    ap.add_argument("--plot_show", action="store_true")
    ap.add_argument("--plot_title", default="GPU PCIe metrics")
    ap.add_argument("--plot_on_exit", action="store_true")
    a = ap.parse_args(argv)
    if a.plot and a.plot_in:
        return plot(a.plot_in, a.plot_out, a.plot_title)
    from skygdr_b200.control import ctl

    sig = ctl.GpuSignals(a.gpu)
    if not sig.available:
        print("NVML is not available on this machine", file=sys.stderr)
        return 1
    header = ctl.GpuSignals.pcie_csv_header() + (",nvlink_tx_GB_s,nvlink_rx_GB_s" if a.nvlink else "")
    if a.out == "-":
        fp = sys.stdout
        fp.write(header + "\n")
    else:
        new = not (a.append and os.path.exists(a.out) and os.path.getsize(a.out) > 0)
        fp = open(a.out, "a" if a.append else "w")
        if new:
            fp.write(header + "\n")
    t0 = time.time()
    try:
        while a.duration_s <= 0 or time.time() - t0 < a.duration_s:
            s = sig.sample_pcie()
            row = s.csv()
            if a.nvlink:
                n = sig.sample_nvlink()
                row += f",{n.tx_gb_s:.3f},{n.rx_gb_s:.3f}"
            fp.write(row + "\n")
            fp.flush()
            if a.live and fp is not sys.stdout:
                print(row, flush=True)
            time.sleep(max(a.interval_ms, 1) / 1000.0)
    except KeyboardInterrupt:
        pass
    if fp is not sys.stdout:
        fp.close()
        if a.plot_on_exit or a.plot:
            plot(a.out, a.plot_out, a.plot_title)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
