"""HBM utilisation logger: memory-controller utilisation x the GPU's peak bandwidth.

    python -m skygdr_b200.cli.bandwidth_usage --gpu 0 --interval_ms 500 --duration_s 0 [--csv] [--out -] [--quiet] [--peak_gbs X]

Columns as in src/tools/bandwidth_usage.py:66-76; minimum interval 50 ms (:55). The peak table knows B200/H200
(the reference's stops at H100); --peak_gbs overrides it, e.g. with the measured copy bandwidth.
"""
from __future__ import annotations

import argparse
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--interval_ms", type=int, default=500)
    ap.add_argument("--duration_s", type=float, default=0.0)
    ap.add_argument("--csv", action="store_true")
    ap.add_argument("--out", default="-")
    ap.add_argument("--quiet", action="store_true")
    ap.add_argument("--peak_gbs", type=float, default=0.0)
    a = ap.parse_args(argv)
    from skygdr_b200.control import ctl

    sig = ctl.GpuSignals(a.gpu, None, a.peak_gbs)
    if not sig.available:
        print("NVML is not available on this machine", file=sys.stderr)
        return 1
    interval = max(a.interval_ms, 50) / 1000.0
    fp = sys.stdout if a.out == "-" else open(a.out, "w")
    fp.write(ctl.GpuSignals.hbm_csv_header() + "\n")
    t0 = time.time()
    try:
        while a.duration_s <= 0 or time.time() - t0 < a.duration_s:
            s = sig.sample_hbm()
            fp.write(s.csv() + "\n")
            fp.flush()
            if not a.quiet and fp is not sys.stdout:
                print(f"mem_util={s.memory_util_pct:.0f}% est_bw={s.estimated_gb_s:.1f} GB/s", flush=True)
            time.sleep(interval)
    except KeyboardInterrupt:
        pass
    if fp is not sys.stdout:
        fp.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
