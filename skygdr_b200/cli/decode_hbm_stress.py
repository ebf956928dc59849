"""decode_hbm_stress <gpu=0> <working_set_mib=32768> <iters=1000>

Streaming b += alpha*a over a half/half working set; models 3 x array bytes per pass and prints the
`HBM stress done:` line of llm_problem_analysis/decode_hbm_stress.cu:95-101,159-178 (GiB/s) plus GB/s.
One persistent launch runs all passes.
"""
from __future__ import annotations

import sys


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    gpu = int(argv[0]) if len(argv) > 0 else 0
    ws_mib = int(argv[1]) if len(argv) > 1 else 32768
    iters = int(argv[2]) if len(argv) > 2 else 1000
    import torch

    from skygdr_b200.ops import Memhog

    torch.cuda.set_device(gpu)
    print(f"gpu={gpu} name={torch.cuda.get_device_name(gpu)} working_set={ws_mib} MiB iters={iters}", flush=True)
    hog = Memhog(f"cuda:{gpu}", gb=ws_mib / 1024.0, op="axpy")
    hog.a.fill_(1.0)
    hog.launch(iters=1)
    hog.result()                        # warm-up pass
    hog.launch(iters=iters, alpha=1e-6)
    r = hog.result()
    checksum = float(hog.b[:: max(1, hog.b.numel() // 4096)].double().sum())
    gib = r["bytes_done"] / 2**30
    print(f"HBM stress done: approx {gib:.2f} GiB in {r['seconds']:.3f} s = {r['gib_s']:.2f} GiB/s ({r['gb_s']:.2f} GB/s)")
    print(f"checksum={checksum:.6e} status={r['status_name']}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
