"""The control loop at work on GPUs, as processes: a protected kv_transfer and a backlogged best-effort bulk transfer that
share one NVLink capacity, under three scheduling arms.

    python benchmarks/scheduler_shared_link.py [--protected-src 0 --besteffort-src 1 --dst 2] [--seconds 6] [--rate 30]
        [--arms always_high,always_low,controlled] [--target-gbps 600] [--capacity-gbps 750] [--out results/shared_link.json]

What shares what: both flows store into pools of the SAME destination GPU, from two different source GPUs, so the
destination's NVLink ingress (one direction of its 18 links) is the capacity they compete for. Each flow has its own source
GPU because its driver is its own process, and two processes whose kernels wait (for credit) must not time-slice one GPU.

Processes per arm: `fabricd` (owns the credit pages under /dev/shm and runs one signal -> policy -> action pass per 1 ms
window), one driver process per flow, and this orchestrator. The drivers register over TCP (`REGISTER <name> <priority>
<target> <kind> link=<link>`), map the page the daemon created (`CreditPage.attach`: cudaHostRegister of the /dev/shm page, so
the kernel reads the daemon's stores directly), and launch the paged transfer kernel (gather from a token-major pool with a
permuted block list, NHD -> HND, peer stores), which checks the page chunk by chunk.

    protected   kv_transfer   priority high, target --target-gbps: Poisson arrivals (--rate per second, seed 0) of requests
                              of 1.2 - 9.4 GB (uniform), served in order; flow time = completion - arrival
    best effort kv_bulk       priority 0, no target: 2 GB transfers back to back for the whole run

Arms: always_high (policy none: nobody is paced), always_low (policy static: the best-effort flow is held to
--low-fraction of the link all the time), controlled (policy target_track: while the protected flow has backlog the best-effort
flow gets what the link has left beside the target, otherwise it is unpaced).

The reference runs the same three arms on its PCIe case study (src/tools/pcie_case_study_analyze.py:140-154) with a Python
controller polling CSV files at 10 Hz (src/tools/pcie_case_study_controller.py:273-352) and reports the protected flow's
finish time; its README quotes 19.4 - 34.4 % lower flow time with scheduling (README.md:74).
"""
import argparse
import json
import os
import statistics
import struct
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

BACKLOG_OFF = 128 + 56          # SkyCreditPage.backlog_bytes (csrc/ctl/credit_page.h)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", default="main", choices=["main", "protected", "besteffort"])
    ap.add_argument("--protected-src", type=int, default=0)
    ap.add_argument("--besteffort-src", type=int, default=1)
    ap.add_argument("--dst", type=int, default=2)
    ap.add_argument("--seconds", type=float, default=6.0)
    ap.add_argument("--rate", type=float, default=30.0, help="protected requests per second (Poisson)")
    ap.add_argument("--min-gb", type=float, default=1.2)
    ap.add_argument("--max-gb", type=float, default=9.4)
    ap.add_argument("--bulk-gb", type=float, default=2.0)
    ap.add_argument("--arms", default="always_high,always_low,controlled")
    ap.add_argument("--target-gbps", type=float, default=600.0)
    ap.add_argument("--capacity-gbps", type=float, default=750.0)
    ap.add_argument("--low-fraction", type=float, default=0.2)
    ap.add_argument("--window-us", type=int, default=1000)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default="results/shared_link.json")
    # internal (driver processes)
    ap.add_argument("--port", type=int, default=0)
    ap.add_argument("--link", default="")
    ap.add_argument("--workdir", default="")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------------------------
# driver processes

def wait_for(path, timeout_s=120.0):
    t0 = time.time()
    while not os.path.exists(path):
        if time.time() - t0 > timeout_s:
            raise TimeoutError(path)
        time.sleep(0.005)
    return open(path).read()


def driver(a):
    import torch

    from skygdr_b200 import ops
    from skygdr_b200._ext import load
    from skygdr_b200.control import FabricClient

    C = load()
    src = a.protected_src if a.role == "protected" else a.besteffort_src
    torch.cuda.set_device(src)
    dev, ddev = torch.device("cuda", src), torch.device("cuda", a.dst)
    assert C.enable_peer_access(src, a.dst), f"no peer access GPU {src} -> GPU {a.dst}"
    geom = ops.KVGeometry()                                   # Qwen3-8B: 36 layers x 8 KV heads x 128, 16-token blocks
    block_bytes = geom.block_elems * 2
    max_blocks = int((a.max_gb if a.role == "protected" else a.bulk_gb) * 1e9 // block_bytes) + 1
    src_pool = ops.PagedKVPool(geom, max_blocks, "nhd", device=dev)
    step = max(1, (1 << 28) // geom.block_elems)
    for i in range(0, max_blocks, step):
        src_pool.data[i:i + step].normal_()
    dst_pool = ops.PagedKVPool(geom, max_blocks, "hnd", device=ddev)
    remote = ops.RemotePool.of(dst_pool)
    g = torch.Generator().manual_seed(a.seed + (1 if a.role == "protected" else 2))
    sb = torch.randperm(max_blocks, generator=g).int().to(dev)
    db = torch.randperm(max_blocks, generator=g).int().to(dev)

    client = FabricClient(port=a.port)
    if a.role == "protected":
        h = client.register("kv_transfer", "high", a.target_gbps, link=a.link)
    else:
        h = client.register("kv_bulk", 0, 0.0, kind="kv_offload", link=a.link)
    page = ops.CreditPage.attach(h.page_path)
    flow = ops.KvTransferFlow(dev, page=page, max_wait_ms=5.0)

    def set_backlog(n):
        struct.pack_into("<Q", h._mm, BACKLOG_OFF, int(n))

    # warm-up: one small transfer (module load, tensor maps), exactness of the path through the daemon's page
    st = flow.transfer_to_completion(src_pool, [remote], sb[:64], db[:64])
    assert st["status"] == 0, st
    torch.cuda.synchronize(ddev)
    assert torch.equal(dst_pool.data[db[:64].long().to(ddev)], ops.reference_transfer(src_pool, sb[:64]).to(ddev)), "transfer not exact"

    open(os.path.join(a.workdir, f"ready_{a.role}"), "w").write("1")
    t0 = float(wait_for(os.path.join(a.workdir, "go")))
    while time.time() < t0:
        time.sleep(0.0005)
    out = {"role": a.role, "src": src, "dst": a.dst, "flow_id": h.flow_id}
    if a.role == "protected":
        import random

        rng = random.Random(a.seed)
        t, reqs = 0.0, []
        while True:
            t += rng.expovariate(a.rate)
            if t >= a.seconds:
                break
            reqs.append((t, rng.uniform(a.min_gb, a.max_gb)))
        recs = []
        for t_arr, gb in reqs:
            now = time.time() - t0
            if now < t_arr:
                time.sleep(t_arr - now)
            nb = max(1, int(gb * 1e9 // block_bytes))
            set_backlog(nb * block_bytes)
            st = flow.transfer_to_completion(src_pool, [remote], sb[:nb], db[:nb])
            set_backlog(0)
            t_done = time.time() - t0
            recs.append({"t_arrival": t_arr, "bytes": st["bytes_done"], "status": st["status"], "launches": st["launches"],
                         "device_ms": st["device_time_ms"], "flow_ms": (t_done - t_arr) * 1e3, "stall_ms": st["stall_ns"] * 1e-6 / max(1, flow.sms)})
        out["requests"] = recs
        open(os.path.join(a.workdir, "protected_done"), "w").write("1")
    else:
        nb = max(1, int(a.bulk_gb * 1e9 // block_bytes))
        set_backlog(1 << 40)
        total, n, launches = 0, 0, 0
        t_begin = time.time()
        while time.time() - t0 < a.seconds:
            st = flow.transfer_to_completion(src_pool, [remote], sb[:nb], db[:nb])
            if st["status"] != 0:
                out["error"] = st
                break
            total += st["bytes_done"]
            n += 1
            launches += st["launches"]
        elapsed = time.time() - t_begin
        set_backlog(0)
        out.update(bytes=total, transfers=n, launches=launches, seconds=elapsed, goodput_gbs=total / elapsed / 1e9)
    usage = h.usage()
    out["page_usage"] = {k: usage[k] for k in ("consumed_bytes", "completed_bytes", "yields", "chunks")}
    client.unregister(h)
    client.close()
    page.close()
    json.dump(out, open(os.path.join(a.workdir, f"result_{a.role}.json"), "w"))
    return 0


# ---------------------------------------------------------------------------------------------------------------
# orchestrator

def pct(xs, q):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(q * len(xs)))] if xs else float("nan")


def pacing_error(log_path, flow_name, window_s):
    """Achieved / granted for a paced flow, from the daemon's window log. A row holds the budget decided for the window that
    begins and the rate measured over the window that just ended, so a budget is set against the rate of the flow's next row.
    Windows in which the flow had nothing to send (no backlog, no bytes) are left out."""
    import csv

    if not os.path.exists(log_path):
        return None
    rows = [r for r in csv.DictReader(open(log_path)) if r["flow"] == flow_name]
    moved = granted = 0.0
    windows = 0
    for cur, nxt in zip(rows, rows[1:]):
        b = float(cur["budget_bytes"])
        got = float(nxt["inst_gbps"]) * 1e9 * window_s
        if b < 0 or (got <= 0 and int(nxt["backlog_bytes"]) == 0):
            continue
        granted += b
        moved += got
        windows += 1
    return {"paced_windows": windows, "granted_gb": granted / 1e9, "moved_gb": moved / 1e9,
            "achieved_over_granted": (moved / granted) if granted else None}


def run_arm(a, arm, workdir):
    from skygdr_b200.control import FabricDaemon

    os.makedirs(workdir, exist_ok=True)
    for f in os.listdir(workdir):
        os.unlink(os.path.join(workdir, f))
    link = f"nvlink:gpu{a.dst}:rx"
    policy = {"always_high": "none", "always_low": "static", "controlled": "target_track"}[arm]
    log = os.path.join(workdir, "fabricd_windows.csv")
    extra = ["--link", f"{link}={a.capacity_gbps}", "--low1_fraction", str(a.low_fraction), "--util_threshold_pct", "0"]
    with FabricDaemon(policy=policy, window_us=a.window_us, lease_ms=600000, log=log, extra=extra) as d:
        procs = []
        for role in ("protected", "besteffort"):
            cmd = [sys.executable, os.path.abspath(__file__), "--role", role, "--port", str(d.port), "--link", link, "--workdir", workdir,
                   "--protected-src", str(a.protected_src), "--besteffort-src", str(a.besteffort_src), "--dst", str(a.dst),
                   "--seconds", str(a.seconds), "--rate", str(a.rate), "--min-gb", str(a.min_gb), "--max-gb", str(a.max_gb),
                   "--bulk-gb", str(a.bulk_gb), "--target-gbps", str(a.target_gbps), "--seed", str(a.seed)]
            procs.append(subprocess.Popen(cmd, stdout=open(os.path.join(workdir, f"{role}.log"), "w"), stderr=subprocess.STDOUT))
        try:
            for role in ("protected", "besteffort"):
                wait_for(os.path.join(workdir, f"ready_{role}"), 300.0)
            open(os.path.join(workdir, "go.tmp"), "w").write(repr(time.time() + 0.5))
            os.rename(os.path.join(workdir, "go.tmp"), os.path.join(workdir, "go"))
            for p in procs:
                p.wait(timeout=a.seconds * 6 + 240)
        finally:
            for p in procs:
                if p.poll() is None:
                    p.kill()
    res = {"arm": arm, "policy": policy}
    for role in ("protected", "besteffort"):
        path = os.path.join(workdir, f"result_{role}.json")
        if not os.path.exists(path):
            res["error"] = f"{role} driver left no result: " + open(os.path.join(workdir, f"{role}.log")).read()[-1500:]
            return res
        res[role] = json.load(open(path))
    reqs = res["protected"]["requests"]
    ok = [r for r in reqs if r["status"] == 0]
    res["summary"] = {
        "requests": len(reqs), "completed": len(ok),
        "flow_ms_p50": pct([r["flow_ms"] for r in ok], 0.5), "flow_ms_p99": pct([r["flow_ms"] for r in ok], 0.99),
        "flow_ms_mean": statistics.fmean([r["flow_ms"] for r in ok]) if ok else float("nan"),
        "device_ms_p50": pct([r["device_ms"] for r in ok], 0.5), "device_ms_p99": pct([r["device_ms"] for r in ok], 0.99),
        "protected_gbs_p50": pct([r["bytes"] / r["device_ms"] / 1e6 for r in ok], 0.5),
        "protected_gb_moved": sum(r["bytes"] for r in ok) / 1e9,
        "besteffort_goodput_gbs": res["besteffort"].get("goodput_gbs"),
        "besteffort_pacing": pacing_error(log, "kv_bulk", a.window_us * 1e-6),
    }
    return res


def main():
    a = parse()
    if a.role != "main":
        a.link = a.link or f"nvlink:gpu{a.dst}:rx"
        return driver(a)
    from skygdr_b200.cli.common import env_info

    base = os.path.join("/dev/shm", f"skygdr_shared_link_{os.getpid()}")
    out = {"config": {k: v for k, v in vars(a).items() if k not in ("role", "port", "link", "workdir")}, "env": env_info(), "arms": {}}
    for arm in a.arms.split(","):
        r = run_arm(a, arm, base)
        out["arms"][arm] = r
        print(arm, json.dumps(r.get("summary", r.get("error"))), flush=True)
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        json.dump(out, open(a.out, "w"), indent=1)
    hi, ctl_ = out["arms"].get("always_high", {}).get("summary"), out["arms"].get("controlled", {}).get("summary")
    if hi and ctl_:
        out["headline"] = {
            "flow_ms_p50_change_pct": 100.0 * (ctl_["flow_ms_p50"] / hi["flow_ms_p50"] - 1.0),
            "flow_ms_p99_change_pct": 100.0 * (ctl_["flow_ms_p99"] / hi["flow_ms_p99"] - 1.0),
            "besteffort_goodput_change_pct": 100.0 * (ctl_["besteffort_goodput_gbs"] / hi["besteffort_goodput_gbs"] - 1.0),
        }
        print("controlled vs always_high:", json.dumps(out["headline"]), flush=True)
        json.dump(out, open(a.out, "w"), indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
