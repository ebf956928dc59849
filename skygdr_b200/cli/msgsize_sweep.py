"""Message-size sweep of the flow load generator.

    python -m skygdr_b200.cli.msgsize_sweep --server_ip 127.0.0.1 --tcp_port 18515 --fabric tcp --iters 2000 --op write
        --msg_sizes 64,4K,64K,1M --out sweep.csv [--warmup_runs 1 --warmup_iters 200 --qd 64 --write_ack 1 ...]

Runs cpu_client once per size (after optional warm-up runs), scrapes its three final lines with the regexes of
src/tools/rdma_msgsize_sweep.py:64-96 and appends one row per size to a CSV with a self-describing header (:138-187).
"""
from __future__ import annotations

import argparse
import csv
import os
import re
import subprocess
import sys
import time

from .common import parse_size

RE_ELAPSED = re.compile(r"\[client\] elapsed=([0-9.]+) s\s+ops=([0-9.]+) ops/s\s+throughput=([0-9.]+) GiB/s")
RE_LAT = re.compile(r"\[client\] latency_us samples=(\d+) p50=([0-9.]+) p90=([0-9.]+) p99=([0-9.]+) p999=([0-9.]+) min=([0-9.]+) max=([0-9.]+)")
FIELDS = ["ts_unix_ms", "msg_bytes", "op", "qd", "qps", "iters", "elapsed_s", "ops_per_s", "throughput_gib_s", "samples", "p50_us",
          "p90_us", "p99_us", "p999_us", "min_us", "max_us", "rc"]


def parse_client_output(text: str) -> dict:
    out = {}
    m = RE_ELAPSED.search(text)
    if m:
        out.update(elapsed_s=float(m.group(1)), ops_per_s=float(m.group(2)), throughput_gib_s=float(m.group(3)))
    m = RE_LAT.search(text)
    if m:
        out.update(samples=int(m.group(1)), p50_us=float(m.group(2)), p90_us=float(m.group(3)), p99_us=float(m.group(4)),
                   p999_us=float(m.group(5)), min_us=float(m.group(6)), max_us=float(m.group(7)))
    return out


def client_cmd(a, msg: int, iters: int):
    from skygdr_b200 import build

    exe = os.path.join(build.build_bin(), "cpu_client")
    # positional tail in the reference's order: qd span pattern align mtu sample max_samples ts_ms ts_out write_ack read_min_qd rd_atomic qps
    fabric = a.ib_dev or a.fabric                 # the reference's --ib_dev names the device; here it names the fabric (sim:<GB/s>, tcp)
    write_ack = 1 if a.write_ack is None else a.write_ack
    return [exe, a.server_ip, str(a.tcp_port), fabric, str(iters), str(msg), a.op, str(a.port), str(a.gid_idx), str(a.qd), str(a.span),
            a.pattern, str(a.align), str(a.mtu), str(a.sample), str(a.max_samples), str(a.ts_ms), a.ts_out, str(write_ack),
            str(16 if a.read_min_qd is None else a.read_min_qd), str(a.rd_atomic or 0), str(a.qps)]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--server_ip", default="-")
    ap.add_argument("--tcp_port", type=int, default=0)
    ap.add_argument("--fabric", default="sim:64")
    ap.add_argument("--iters", type=int, default=2000)
    ap.add_argument("--op", default="write", choices=["write", "read"])
    ap.add_argument("--qd", type=int, default=64)
    ap.add_argument("--qps", type=int, default=1)
    ap.add_argument("--span", default="0")
    ap.add_argument("--pattern", default="random")
    ap.add_argument("--align", type=int, default=256)
    ap.add_argument("--sample", type=int, default=1)
    ap.add_argument("--write_ack", type=int, choices=[0, 1], default=None)
    # the rest of the reference's flag set (src/tools/rdma_msgsize_sweep.py:101-127), passed through to the client's positional tail
    ap.add_argument("--cpu_client", default="", help="accepted for compatibility; the in-tree client is used")
    ap.add_argument("--ib_dev", default="", help="fabric name: sim:<GB/s> or tcp (takes the place of the verbs device)")
    ap.add_argument("--port", type=int, default=1)
    ap.add_argument("--gid_idx", type=int, default=0)
    ap.add_argument("--mtu", type=int, default=1024)
    ap.add_argument("--max_samples", type=int, default=0)
    ap.add_argument("--ts_ms", type=int, default=0)
    ap.add_argument("--ts_out", default="")
    ap.add_argument("--write_ack_batch", type=int, default=None, help="deprecated in the reference too; ignored")
    ap.add_argument("--read_min_qd", type=int, default=None)
    ap.add_argument("--rd_atomic", type=int, default=None)
    ap.add_argument("--msg_sizes", default="64,4K,64K,1M")
    ap.add_argument("--warmup_iters", type=int, default=200)
    ap.add_argument("--warmup_runs", type=int, default=1)
    ap.add_argument("--warmup_sleep_ms", type=int, default=0)
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    new = not (os.path.exists(a.out) and os.path.getsize(a.out) > 0)
    with open(a.out, "a", newline="") as fp:
        w = csv.DictWriter(fp, fieldnames=FIELDS)
        if new:
            w.writeheader()
        for tok in a.msg_sizes.split(","):
            msg = parse_size(tok.strip())
            for _ in range(a.warmup_runs):
                subprocess.run(client_cmd(a, msg, a.warmup_iters), capture_output=True, text=True)
                time.sleep(a.warmup_sleep_ms / 1000.0)
            r = subprocess.run(client_cmd(a, msg, a.iters), capture_output=True, text=True)
            row = {"ts_unix_ms": int(time.time() * 1000), "msg_bytes": msg, "op": a.op, "qd": a.qd, "qps": a.qps, "iters": a.iters, "rc": r.returncode}
            row.update(parse_client_output(r.stdout))
            w.writerow(row)
            fp.flush()
            print(f"msg={msg} rc={r.returncode} throughput_gib_s={row.get('throughput_gib_s')} p50_us={row.get('p50_us')}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
