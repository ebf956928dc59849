"""gpu_pcie_memcpy: chunked host<->device copy task with progress reporting.

    python -m skygdr_b200.cli.gpu_pcie_memcpy --device=0 --seconds=60 --dir=h2d|d2h --bytes=SIZE|--chunk_mb=128 --streams=8
        --batch=8 --inflight=8 --pinned=1 --report_ms=1000 --total_bytes=0 --max_outstanding_bytes=0 --progress_ms=..
        --progress_smooth_windows=5 --progress_out=PATH --duty_on_ms=0 --duty_off_ms=0 [--credit_page=/dev/shm/...]

Flags, `[pcie]` stdout lines and the progress CSV follow src/gpu_be_pcie_memcpy_task.cu:53-156,261,372-374.
`--seconds=0 --total_bytes=N` is the finite "restore window" mode the policy loop uses
(src/tools/pcie_case_study_controller.py:205-221). The native worker is skygdr_b200/csrc/kernels/pcie_task.cpp.
"""
from __future__ import annotations

import argparse
import signal
import time

from .common import parse_size


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--seconds", type=float, default=60.0)
    ap.add_argument("--dir", default="d2h", choices=["h2d", "d2h"])
    ap.add_argument("--bytes", default=None)
    ap.add_argument("--chunk_mb", type=int, default=128)
    ap.add_argument("--streams", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--inflight", type=int, default=8)
    ap.add_argument("--pinned", type=int, default=1)
    ap.add_argument("--report_ms", type=int, default=1000)
    ap.add_argument("--total_bytes", default="0")
    ap.add_argument("--max_outstanding_bytes", default="0")
    ap.add_argument("--progress_ms", type=int, default=0)
    ap.add_argument("--progress_smooth_windows", type=int, default=5)
    ap.add_argument("--progress_out", default="")
    ap.add_argument("--duty_on_ms", type=int, default=0)
    ap.add_argument("--duty_off_ms", type=int, default=0)
    ap.add_argument("--credit_page", default="", help="path of a credit page created by fabricd for this flow")
    return ap


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    from skygdr_b200._ext import load

    C = load()
    cfg = C.PcieTaskConfig()
    cfg.device, cfg.h2d = a.device, a.dir == "h2d"
    cfg.chunk_bytes = parse_size(a.bytes) if a.bytes else a.chunk_mb << 20
    cfg.streams, cfg.batch, cfg.inflight, cfg.pinned = a.streams, a.batch, a.inflight, bool(a.pinned)
    cfg.seconds = a.seconds
    cfg.total_bytes = parse_size(a.total_bytes)
    cfg.max_outstanding_bytes = parse_size(a.max_outstanding_bytes)
    cfg.progress_ms = a.progress_ms or a.report_ms
    cfg.smooth_windows = a.progress_smooth_windows
    cfg.duty_on_ms, cfg.duty_off_ms = a.duty_on_ms, a.duty_off_ms
    page = None
    if a.credit_page:
        from skygdr_b200.ops.flow import CreditPage

        page = CreditPage.attach(a.credit_page)
        cfg.set_credit_page(page.host_ptr)
    task = C.PcieTask(cfg)
    stop = {"flag": False}
    signal.signal(signal.SIGINT, lambda *_: (stop.__setitem__("flag", True), task.stop()))
    fp = open(a.progress_out, "w") if a.progress_out else None
    if fp:
        fp.write(C.PcieTask.csv_header() + "\n")
        fp.flush()
    if not task.start():
        print(f"[pcie] failed to start: {task.error()}")
        return 1
    seen = 0
    last_print = 0.0
    while task.running:
        time.sleep(min(0.05, cfg.progress_ms / 1000.0))
        rows = task.rows()
        for r in rows[seen:]:
            if fp:
                fp.write(r.csv() + "\n")
                fp.flush()
            if r.elapsed_ms - last_print >= a.report_ms or r.done:
                print(task.stdout_line(r), flush=True)
                last_print = r.elapsed_ms
        seen = len(rows)
    task.join()
    rows = task.rows()
    for r in rows[seen:]:
        if fp:
            fp.write(r.csv() + "\n")
        print(task.stdout_line(r), flush=True)
    if fp:
        fp.close()
    p = task.progress()
    print(f"[pcie] done dir={a.dir} completed_bytes={p.completed_bytes} elapsed_s={p.elapsed_ms / 1e3:.3f} avg_bw_gib_s={p.avg_bw_gib_s:.3f} "
          f"avg_bw_gb_s={p.avg_bw_gib_s * 1.073741824:.3f}")
    if task.error():
        print(f"[pcie] error: {task.error()}")
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
