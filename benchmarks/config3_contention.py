"""Decode / NVLink / HBM contention on one GPU, with and without scheduling.

    python benchmarks/config3_contention.py [--decode-gpu 1 --src-gpu 0] [--out results/config3.json] [--ref]

On the decode GPU: paged GQA decode attention (32 query / 8 KV heads, head_dim 128, bf16, batch 64, context lengths
log-normal with median 8k clipped to 1k-32k, 36 layers per step). Against it: an inbound 4 GB KV transfer from the
source GPU over NVLink (landing in the decode GPU's HBM) and the memhog best-effort task at 50 % HBM duty.
Phases, as in the reference's colocation harness (alone / alone / overlapped:
llm_problem_analysis/run_hbm_kv_overlap_bench.sh:120-191, final_run_vllm_decode_kv_colocation_bench.sh:251-341):

  decode_alone, transfer_alone, memhog_alone
  contended_unscheduled : all three at once, nobody paced
  contended_scheduled   : the control core (C++ DaemonCore, `target_track`, 2 ms windows) sees decode as the protected
                          flow (its achieved KV-read rate against the uncontended rate), the transfer as a flow with a
                          bandwidth goal, memhog as best effort, and writes byte grants into the credit pages that the
                          memhog and transfer kernels check per chunk.
Reported: decode tokens/s (and its ratio to uncontended), transfer time, memhog GB/s, per phase. Device-timed.
"""
import argparse
import json
import math
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from skygdr_b200 import ops  # noqa: E402
from skygdr_b200._ext import load  # noqa: E402
from skygdr_b200.cli.common import env_info  # noqa: E402
from skygdr_b200.control import ctl  # noqa: E402


class DecodeLoop:
    """36 attention layers per step over a fixed batch; KV bytes read per step are known exactly."""

    def __init__(self, dev, batch, seed, layers=36):
        self.dev, self.layers, self.batch = dev, layers, batch
        rng = ctl.Rng(seed)
        ctx = [int(rng.lognormal(8192, 0.6, 1024, 32768)) for _ in range(batch)]
        self.ctx = torch.tensor(ctx, dtype=torch.int32, device=dev)
        self.geom = ops.KVGeometry(layers=1, kv_heads=8)        # one layer's pages are reused by all 36 passes: same traffic, 1/36 of the memory
        nblk = sum((c + 15) // 16 for c in ctx) + 1
        self.pool = ops.PagedKVPool(self.geom, nblk, "hnd", device=dev)
        for i in range(0, nblk, 4096):
            self.pool.data[i:i + 4096].normal_()
        mb = (max(ctx) + 15) // 16
        self.table = torch.zeros((batch, mb), dtype=torch.int32, device=dev)
        perm = (torch.randperm(nblk - 1) + 1).int()
        o = 0
        for b, c in enumerate(ctx):
            nb = (c + 15) // 16
            self.table[b, :nb] = perm[o:o + nb].to(dev)
            o += nb
        self.q = torch.randn((batch, 32, 128), dtype=torch.bfloat16, device=dev)
        self.out = torch.empty_like(self.q)
        self.attn = ops.PagedAttention(dev, batch, 32, 8, max_ctx=max(ctx), chunk_tokens=1024, impl="tc")
        self.bytes_per_step = sum(ctx) * 8 * 128 * 2 * 2 * layers
        self.stream = torch.cuda.Stream(dev, priority=-1)
        self.max_ctx = max(ctx)

    def step(self):
        for _ in range(self.layers):
            self.attn(self.q, self.pool, 0, self.table, self.ctx, max_ctx=self.max_ctx, out=self.out)

    def run(self, seconds, on_step=None):
        """Runs steps for about `seconds`; returns (steps, device seconds)."""
        with torch.cuda.stream(self.stream):
            self.step()
            self.stream.synchronize()
            steps, t_dev = 0, 0.0
            t0 = time.perf_counter()
            while time.perf_counter() - t0 < seconds:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                self.step()
                e1.record(self.stream)
                e1.synchronize()
                t_dev += e0.elapsed_time(e1) * 1e-3
                steps += 1
                if on_step:
                    on_step(steps)
        return steps, t_dev


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--decode-gpu", type=int, default=1)
    ap.add_argument("--src-gpu", type=int, default=0)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seconds", type=float, default=3.0)
    ap.add_argument("--transfer-gb", type=float, default=4.0)
    ap.add_argument("--memhog-gb", type=float, default=8.0)
    ap.add_argument("--transfer-target-gbps", type=float, default=200.0)
    ap.add_argument("--out", default="results/config3.json")
    a = ap.parse_args()
    C = load()
    ddev, sdev = torch.device("cuda", a.decode_gpu), torch.device("cuda", a.src_gpu)
    assert a.decode_gpu != a.src_gpu and C.enable_peer_access(a.src_gpu, a.decode_gpu) and C.enable_peer_access(a.decode_gpu, a.src_gpu)
    res = {"env": env_info(), "config": vars(a), "phases": {}}
    dec = DecodeLoop(ddev, a.batch, seed=0)
    # inbound transfer: source pool on the other GPU, destination pool in the decode GPU's HBM
    geom = ops.KVGeometry()
    nb = int(a.transfer_gb * 1e9 / (geom.block_elems * 2))
    src = ops.PagedKVPool(geom, nb, "nhd", device=sdev)
    for i in range(0, nb, 256):
        src.data[i:i + 256].normal_()
    dst = ops.PagedKVPool(geom, nb, "hnd", device=ddev)
    sp, dp = torch.randperm(nb).int().to(sdev), torch.randperm(nb).int().to(sdev)
    t_page = ops.CreditPage(flow_id=2, unlimited=True)
    t_flow = ops.KvTransferFlow(sdev, page=t_page, max_wait_ms=20.0)
    h_page = ops.CreditPage(flow_id=3, unlimited=True)
    sms = torch.cuda.get_device_properties(ddev).multi_processor_count
    hog = ops.Memhog(ddev, gb=a.memhog_gb, op="axpy", ctas=sms, page=h_page)       # one CTA per SM: leaves room for decode CTAs
    hog_stream = torch.cuda.Stream(ddev, priority=0)

    def transfer_once():
        with torch.cuda.device(sdev):
            st = t_flow.transfer_to_completion(src, [ops.RemotePool.of(dst)], sp, dp)
        return st

    def hog_run(seconds):
        with torch.cuda.stream(hog_stream):
            hog.launch(iters=0, seconds=seconds, duty_on_ms=2.0, duty_off_ms=2.0, max_wait_ms=50.0)
        return hog

    # ---- alone ----
    steps, t = dec.run(a.seconds)
    base_tok_s = steps * a.batch / t
    base_kv_gbs = steps * dec.bytes_per_step / t / 1e9
    res["phases"]["decode_alone"] = {"tok_s": base_tok_s, "ms_per_step": 1e3 * t / steps, "kv_read_gbs": base_kv_gbs}
    transfer_once()
    st = transfer_once()
    res["phases"]["transfer_alone"] = {"ms": st["device_time_ms"], "gbs": st["bytes_done"] / st["device_time_ms"] / 1e6}
    hog_run(1.0)
    r = hog.result()
    res["phases"]["memhog_alone_50pct_duty"] = {"gbs": r["gb_s"], "seconds": r["seconds"]}

    def contended(scheduled: bool):
        t_page.set_unlimited(); h_page.set_unlimited()
        stop = threading.Event()
        xfer_ms = []

        def xfer_loop():
            time.sleep(0.2)
            while not stop.is_set():
                st = transfer_once()
                xfer_ms.append(st["device_time_ms"])
                time.sleep(0.25)

        core = None
        ctl_thread = None
        progress = {"decode_bytes": 0}
        if scheduled:
            cfg = ctl.DaemonConfig()
            cfg.page_dir, cfg.capacity_gbps, cfg.window_ns, cfg.policy = "", 6400.0, 2_000_000, "target_track"
            cfg.lease_ns = 3600 * 10**9
            cfg.pcfg.enter_ratio, cfg.pcfg.exit_ratio, cfg.pcfg.util_threshold_pct = 0.97, 0.99, 0.0
            cfg.pcfg.min_be_fraction = 0.01
            core = ctl.DaemonCore(cfg)
            core.handle_line(f"REGISTER decode high {base_kv_gbs * 0.98:.1f} other", time.perf_counter_ns())
            core.handle_line(f"REGISTER kv_transfer normal {a.transfer_target_gbps} kv_transfer", time.perf_counter_ns())
            core.handle_line("REGISTER memhog besteffort 0 best_effort", time.perf_counter_ns())

            def control_loop():
                # mirror the daemon's pages <-> the device-visible pages of the two kernels, every window
                hog_base = h_page.read()["consumed_bytes"]
                granted_hog = hog_base
                while not stop.is_set():
                    now = time.perf_counter_ns()
                    core.report_usage(1, progress["decode_bytes"], progress["decode_bytes"], 1 << 40)
                    tu, hu = t_page.read(), h_page.read()
                    core.report_usage(2, tu["consumed_bytes"], tu["completed_bytes"], 1 << 30)
                    core.report_usage(3, hu["consumed_bytes"], hu["completed_bytes"], 1 << 40)
                    core.step_window(now)
                    f3 = core.page_fields(3)
                    if f3["unlimited"]:
                        h_page.set_unlimited()
                    else:
                        h_page.grant(int(f3["granted_bytes"]), unlimited=False)
                    time.sleep(0.002)

            ctl_thread = threading.Thread(target=control_loop, daemon=True)
        th = threading.Thread(target=xfer_loop, daemon=True)
        hog_run(a.seconds + 1.0)
        th.start()
        if ctl_thread:
            ctl_thread.start()

        def on_step(n):
            progress["decode_bytes"] = n * dec.bytes_per_step

        steps, t = dec.run(a.seconds, on_step)
        stop.set()
        th.join()
        if ctl_thread:
            ctl_thread.join()
        h_page.grant(0, unlimited=True)
        r = hog.result()
        return {"tok_s": steps * a.batch / t, "vs_uncontended": steps * a.batch / t / base_tok_s, "ms_per_step": 1e3 * t / steps,
                "transfer_ms": xfer_ms, "transfer_ms_mean": sum(xfer_ms) / len(xfer_ms) if xfer_ms else None, "memhog_gbs": r["gb_s"],
                "memhog_status": r["status_name"]}

    res["phases"]["contended_unscheduled"] = contended(False)
    res["phases"]["contended_scheduled"] = contended(True)
    os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
    json.dump(res, open(a.out, "w"), indent=1)
    print(json.dumps(res["phases"], indent=1))


if __name__ == "__main__":
    main()
