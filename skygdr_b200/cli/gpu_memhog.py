"""gpu_memhog: best-effort HBM task.

    python -m skygdr_b200.cli.gpu_memhog --device=0 --gb=16 --op=rw|read|write|copy|axpy --seconds=60 --iters=100
                                         [--blocks=N --threads=256 --duty_on_ms=0 --duty_off_ms=0 --streams=1 --vec=4]

Flags and the `[memhog]` output lines follow src/gpu_be_memhog_task.cu:142-201,354-358. One persistent launch
replaces the reference's host loop of launches; `--duty_on_ms/--duty_off_ms` give an in-kernel duty cycle, and
`--credit` gates it by a flow's credit page. `--streams` and `--vec` are accepted for compatibility (the kernel
is always 16-byte vectorised and one launch fills the GPU).
"""
from __future__ import annotations

import argparse
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--gb", type=float, default=16.0)
    ap.add_argument("--blocks", type=int, default=0)
    ap.add_argument("--threads", type=int, default=256)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--seconds", type=float, default=60.0)
    ap.add_argument("--op", default="rw", choices=["rw", "read", "write", "copy", "axpy"])
    ap.add_argument("--streams", type=int, default=1)
    ap.add_argument("--vec", type=int, default=4)
    ap.add_argument("--duty_on_ms", type=float, default=0.0)
    ap.add_argument("--duty_off_ms", type=float, default=0.0)
    a = ap.parse_args(argv)
    import torch

    from skygdr_b200.ops import Memhog

    torch.cuda.set_device(a.device)
    hog = Memhog(f"cuda:{a.device}", gb=a.gb, op=a.op, ctas=a.blocks or None, threads=a.threads)
    t0 = time.time()
    if a.seconds > 0:
        hog.launch(iters=0, seconds=a.seconds, duty_on_ms=a.duty_on_ms, duty_off_ms=a.duty_off_ms)
    else:                                   # exactly one measured pass set, like the reference's seconds<=0 mode
        hog.launch(iters=max(1, a.iters), duty_on_ms=a.duty_on_ms, duty_off_ms=a.duty_off_ms)
    r = hog.result()
    wall = time.time() - t0
    print(f"[memhog] device={a.device} op={a.op} gb={a.gb:.2f} blocks={hog.ctas} threads={a.threads} duty_on_ms={a.duty_on_ms} "
          f"duty_off_ms={a.duty_off_ms} status={r['status_name']}")
    print(f"[memhog] bytes={r['bytes_done']} kernel_s={r['seconds']:.6f} bw_gib_s={r['gib_s']:.2f} bw_gb_s={r['gb_s']:.2f}")
    print(f"[memhog] wall_s={wall:.3f}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
