"""Prefill / decode disaggregation emulation: prefill GPUs run prompts, hand their paged KV to decode GPUs over
NVLink with the credit-gated transfer kernel, while a background kv_offload streams KV to pinned host memory.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        benchmarks/config4_pd_disagg.py --prefill-gpus 4 --decode-gpus 4 [--arm controlled|always_high|always_low]
        [--rate 4 --duration 20] [--offload-gbps 24] [--layers 36] [--out results/config4.json]

Requests (same seed on every rank): Poisson arrivals, input lengths log-normal (median 16k, clipped to 64k), output
lengths uniform 128-1024 (scaled by --out-scale). Request i is prefilled on prefill rank i % P and decoded on decode
rank i % D, in one of that rank's KV slots. Per request:

  arrival -> (queue) -> prefill (this package's GEMMs / norm / RoPE+append and its tcgen05 prefill attention over the paged pool)
          -> kv_transfer: paged gather + token-major -> head-major + peer stores into the decode rank's pool; the
             kernel's last CTA publishes `first_token + 1` in the request's ready flag (release, system scope)
          -> decode rank sees the flag (acquire) and adds the sequence to its running batch -> first decode step = TTFT

Arms (the reference's three: src/tools/pcie_case_study_analyze.py:140-154): `always_high` = offload unpaced;
`always_low` = offload statically throttled to a quarter of its offered rate; `controlled` = `target_track` with 2 ms windows
cuts the offload's byte grants while a hand-off is in flight and releases them afterwards. The control side of the controlled
arm is a `fabricd` process (`--daemon`, the default): rank 0 starts it, every prefill rank registers its two flows over TCP on
a link of its own (`gpu<r>`), maps the pages the daemon created under /dev/shm, and its transfer kernel and offload worker
read the daemon's grants from there. `--no-daemon` keeps the control core inside each prefill rank's process instead. Reported per arm: kv_transfer flow time p50/p99 (prefill done -> last byte visible), mean TTFT,
decode tokens/s, offload GB/s. Times across ranks use one wall clock (single node); transfer times are also device-timed.
"""
import argparse
import json
import os
import struct
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from skygdr_b200 import ops  # noqa: E402
from skygdr_b200._ext import load  # noqa: E402
from skygdr_b200.cli.common import env_info  # noqa: E402
from skygdr_b200.control import ctl  # noqa: E402
from skygdr_b200.models import Qwen3Config, Qwen3Decoder, Qwen3Weights  # noqa: E402
from skygdr_b200.parallel.symm import SymmetricHeap  # noqa: E402


def set_backlog(handle, n):
    """Writes a flow's backlog into the usage half of its credit page (SkyCreditPage.backlog_bytes, csrc/ctl/credit_page.h)."""
    struct.pack_into("<Q", handle._mm, 128 + 56, int(n))


def make_requests(a, P, D):
    rng = ctl.Rng(a.seed)
    reqs, t = [], 0.0
    slots_used = [0] * D
    while True:
        t += rng.exponential(a.rate)
        if t >= a.duration:
            break
        n_in = int(rng.lognormal(a.median_in, 0.7, 1024, a.max_in))
        n_out = max(4, int(rng.uniform_range(128, 1024) * a.out_scale))
        i = len(reqs)
        d = i % D
        reqs.append(dict(id=i, t=t, n_in=n_in, n_out=n_out, prefill=i % P, decode=d, slot=slots_used[d] % a.slots, gen=slots_used[d] // a.slots))
        slots_used[d] += 1
    return reqs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prefill-gpus", type=int, default=1)
    ap.add_argument("--decode-gpus", type=int, default=1)
    ap.add_argument("--arm", default="controlled", choices=["controlled", "always_high", "always_low"])
    ap.add_argument("--rate", type=float, default=2.0)
    ap.add_argument("--duration", type=float, default=10.0)
    ap.add_argument("--median-in", type=int, default=16384)
    ap.add_argument("--max-in", type=int, default=65536)
    ap.add_argument("--out-scale", type=float, default=0.25)
    ap.add_argument("--offload-gbps", type=float, default=24.0)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--slots", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default="results/config4.json")
    ap.add_argument("--daemon", dest="daemon", action="store_true", default=True)
    ap.add_argument("--no-daemon", dest="daemon", action="store_false")
    a = ap.parse_args()
    C = load()
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    P, D = a.prefill_gpus, a.decode_gpus
    assert world == P + D
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    store = dist.distributed_c10d._get_default_store()
    cfg = Qwen3Config(layers=a.layers)
    geom = cfg.geometry
    reqs = make_requests(a, P, D)
    slot_blocks = geom.blocks_for(a.max_in + 1024 + 16)
    is_prefill = rank < P

    # every rank allocates the same heap layout; only decode ranks use the pool, only their flags are written
    pool_bytes = a.slots * slot_blocks * geom.block_elems * 2
    heap = SymmetricHeap((pool_bytes if not is_prefill else 4096) + 65536, rank, world, dev)
    # offsets must match on all ranks: put the flags first, then the pool
    heap.alloc("flags", 16384)
    heap.alloc("pool", pool_bytes, local=not is_prefill)
    dist.barrier()
    weights = Qwen3Weights(cfg, dev, seed=1)
    result = {}
    daemon = None
    if a.arm == "controlled" and a.daemon:
        from skygdr_b200.control import FabricClient, FabricDaemon

        if rank == 0:
            # one link per prefill GPU: its hand-off and its offload compete for that GPU (copy engines, HBM), not across GPUs
            extra = [x for r in range(P) for x in ("--link", f"gpu{r}={a.offload_gbps + 40.0}")] + ["--util_threshold_pct", "0"]
            daemon = FabricDaemon(policy="target_track", window_us=2000, lease_ms=3600 * 1000, extra=extra)
            store.set("fabricd_port", str(daemon.port))
        dist.barrier()
        fabricd_port = int(store.get("fabricd_port").decode())

    if is_prefill:
        mine = [r for r in reqs if r["prefill"] == rank]
        nblk = geom.blocks_for(a.max_in) + 1
        pool = ops.PagedKVPool(geom, nblk, "nhd", device=dev)
        scratch_dec = ops.PagedKVPool(geom, 2, "hnd", device=dev)
        eng = Qwen3Decoder(cfg, weights, scratch_dec, max_batch=1, max_ctx=256, attn_chunk=128)
        client = None
        if a.arm == "controlled" and a.daemon:
            client = FabricClient(port=fabricd_port)
            h_t = client.register(f"kv_transfer{rank}", "high", 40.0, kind="kv_transfer", link=f"gpu{rank}")
            h_o = client.register(f"kv_offload{rank}", 0, 0.0, kind="kv_offload", link=f"gpu{rank}")
            t_page, o_page = ops.CreditPage.attach(h_t.page_path), ops.CreditPage.attach(h_o.page_path)
        else:
            t_page = ops.CreditPage(flow_id=1, unlimited=True)
            o_page = ops.CreditPage(flow_id=2, unlimited=True)
        flow = ops.KvTransferFlow(dev, page=t_page, max_wait_ms=20.0)
        # background offload of "prefix KV": chunked async copies, credit-gated
        pc = C.PcieTaskConfig()
        pc.device, pc.h2d, pc.chunk_bytes, pc.streams, pc.batch, pc.inflight = local, False, 32 << 20, 4, 2, 4
        pc.seconds, pc.progress_ms = a.duration + 60.0, 100
        if client is not None:
            # the daemon leaves an unprotected flow unpaced while nothing needs protecting; the emulated offload only ever has
            # its offered rate to send, which a duty cycle of the copy loop stands for (the link moves about 55 GB/s)
            duty = max(0.05, min(1.0, a.offload_gbps / 55.0))
            pc.duty_on_ms, pc.duty_off_ms = max(1, int(round(20 * duty))), max(0, int(round(20 * (1 - duty))))
            pc.max_outstanding_bytes = 64 << 20               # a short queue, so that the off phase really is off
        pc.set_credit_page(o_page.host_ptr)
        task = C.PcieTask(pc)
        task.setup()
        stop = threading.Event()
        in_flight = {"bytes": 0}
        if a.arm == "always_low":
            pacer = ops.LocalPacer(o_page, a.offload_gbps * 0.25, window_ms=2.0).start(base=0)
        elif a.arm == "always_high":
            pacer = ops.LocalPacer(o_page, a.offload_gbps, window_ms=2.0).start(base=0)       # offered rate, never cut
        elif client is not None:
            pacer = None
            set_backlog(h_o, 1 << 40)                         # the offload is always backlogged
        else:
            pacer = None
            dc = ctl.DaemonConfig()
            dc.page_dir, dc.capacity_gbps, dc.window_ns, dc.policy = "", a.offload_gbps + 40.0, 2_000_000, "target_track"
            dc.lease_ns = 3600 * 10**9          # in-process flows: no lease renewals needed for the length of a run
            dc.pcfg.util_threshold_pct = 0.0
            core = ctl.DaemonCore(dc)
            core.handle_line("REGISTER kv_transfer high 40 kv_transfer", time.perf_counter_ns())
            core.handle_line("REGISTER kv_offload besteffort 0 kv_offload", time.perf_counter_ns())

            def control():
                # The daemon core decides (unlimited / a byte grant for the offload); this loop turns "unlimited" into the
                # offload's offered rate, since the emulated offload never has more than that to send.
                granted, t_prev = 0.0, time.perf_counter()
                while not stop.is_set():
                    now = time.perf_counter()
                    dt, t_prev = now - t_prev, now
                    tu, ou = t_page.read(), o_page.read()
                    core.report_usage(1, tu["consumed_bytes"], tu["completed_bytes"], in_flight["bytes"])
                    core.report_usage(2, ou["consumed_bytes"], ou["completed_bytes"], 1 << 40)
                    core.step_window(time.perf_counter_ns())
                    f = core.page_fields(2)
                    rate = a.offload_gbps if f["unlimited"] else min(a.offload_gbps, f["budget_per_window"] / 0.002 / 1e9)
                    granted = min(max(granted, float(ou["consumed_bytes"])) + rate * 1e9 * dt, ou["consumed_bytes"] + rate * 1e9 * 0.006 + (8 << 20))
                    o_page.grant(int(granted), unlimited=False)
                    time.sleep(0.002)

            threading.Thread(target=control, daemon=True).start()
        # one small prompt before the clock starts: library initialisation and allocator growth are not part of TTFT
        wn = 4096
        eng.prefill(torch.randint(0, cfg.vocab, (wn,), device=dev), [wn], torch.arange(1, geom.blocks_for(wn) + 1, dtype=torch.int32, device=dev).view(1, -1), pool=pool)
        torch.cuda.synchronize(dev)
        dist.barrier()
        t0 = time.perf_counter()
        task.start()
        recs = []
        for r in mine:
            now = time.perf_counter() - t0
            if now < r["t"]:
                time.sleep(r["t"] - now)
            t_start = time.perf_counter() - t0
            nb = geom.blocks_for(r["n_in"])
            table = torch.arange(1, nb + 1, dtype=torch.int32, device=dev)[torch.randperm(nb, device=dev)].view(1, nb)
            ids = torch.randint(0, cfg.vocab, (r["n_in"],), device=dev)
            logits = eng.prefill(ids, [r["n_in"]], table, pool=pool)
            first = int(logits[0].float().argmax())
            torch.cuda.synchronize(dev)
            t_prefill = time.perf_counter() - t0
            # the decode slot must have been released by its previous occupant
            if r["gen"] > 0:
                store.wait([f"free/{r['decode']}/{r['slot']}/{r['gen'] - 1}"])
            drank = P + r["decode"]
            dst_blocks = (torch.arange(nb, dtype=torch.int32, device=dev) + r["slot"] * slot_blocks)
            hnd = ops.PagedKVPool(geom, 1, "hnd", device=dev)       # geometry carrier for the strides
            remote = ops.RemotePool(heap.ptr("pool", drank), (geom.block_elems, 2 * geom.page_elems, geom.page_elems), geom.kv_heads,
                                    0, heap.ptr("flags", drank, 4 * r["id"]))
            in_flight["bytes"] = nb * geom.block_elems * 2
            if client is not None:
                set_backlog(h_t, in_flight["bytes"])          # what the daemon reads as "the protected flow has work"
            flow.seq = first                                         # the ready flag carries first_token + 1
            st = flow.transfer_to_completion(pool, [remote], table.view(-1), dst_blocks)
            in_flight["bytes"] = 0
            if client is not None:
                set_backlog(h_t, 0)
            t_done = time.perf_counter() - t0
            recs.append(dict(id=r["id"], n_in=r["n_in"], t_arrival=r["t"], t_start=t_start, t_prefill_done=t_prefill, t_transfer_done=t_done,
                             flow_time_ms=(t_done - t_prefill) * 1e3, transfer_device_ms=st["device_time_ms"], launches=st["launches"],
                             gbs=st["bytes_done"] / max(st["device_time_ms"], 1e-6) / 1e6))
        stop.set()
        task.stop()
        task.join()
        if pacer:
            pacer.stop()
        result = {"role": "prefill", "requests": recs, "offload_gb_s": task.progress().avg_bw_gib_s * 1.073741824,
                  "control": "fabricd process" if client is not None else "in-process"}
        if client is not None:
            result["offload_page"] = {k: h_o.usage()[k] for k in ("consumed_bytes", "completed_bytes")}
            client.close()
    else:
        drank = rank - P
        mine = [r for r in reqs if r["decode"] == drank]
        pool = ops.PagedKVPool(geom, a.slots * slot_blocks, "hnd", device=dev, data=heap.local_tensor("pool", (pool_bytes // 2,), torch.bfloat16))
        flags = heap.local_tensor("flags", (4096,), torch.int32)
        eng = Qwen3Decoder(cfg, weights, pool, max_batch=a.slots, max_ctx=a.max_in + 1024 + 16, attn_chunk=1024)
        eng.set_batch(torch.zeros(1, dtype=torch.int32, device=dev), torch.full((1,), 8, dtype=torch.int32, device=dev),
                      torch.zeros((1, 1), dtype=torch.int32, device=dev))
        eng.step(b=1, max_ctx=64, advance=False)            # warm-up step on block 0
        torch.cuda.synchronize(dev)
        dist.barrier()
        t0 = time.perf_counter()
        pending = {r["id"]: r for r in mine}
        active = {}                     # slot -> dict(req, pos, left, t_first)
        recs, tokens, t_busy = [], 0, 0.0
        flags_host = torch.zeros(4096, dtype=torch.int32).pin_memory()
        side = torch.cuda.Stream(dev)
        t_end = a.duration + 120.0
        while (pending or active) and time.perf_counter() - t0 < t_end:
            with torch.cuda.stream(side):
                flags_host.copy_(flags, non_blocking=True)
            side.synchronize()
            for rid in [i for i in pending if int(flags_host[i]) > 0]:
                r = pending.pop(rid)
                active[r["slot"]] = dict(req=r, pos=r["n_in"], left=r["n_out"], tok=int(flags_host[rid]) - 1, t_seen=time.perf_counter() - t0, t_first=None)
            if not active:
                time.sleep(0.0005)
                continue
            slots = sorted(active)
            b = len(slots)
            ids = torch.tensor([active[s]["tok"] for s in slots], dtype=torch.int32, device=dev)
            pos = torch.tensor([active[s]["pos"] for s in slots], dtype=torch.int32, device=dev)
            mb = max(geom.blocks_for(active[s]["pos"] + 1) for s in slots)
            table = torch.stack([torch.arange(mb, dtype=torch.int32, device=dev) + s * slot_blocks for s in slots])
            ts = time.perf_counter()
            eng.set_batch(ids, pos, table)
            out = eng.step(b=b, max_ctx=int(pos.max()) + 1, advance=False).tolist()
            torch.cuda.synchronize(dev)
            now = time.perf_counter()
            t_busy += now - ts
            tokens += b
            for s, tok in zip(slots, out):
                st = active[s]
                if st["t_first"] is None:
                    st["t_first"] = now - t0
                st["tok"], st["pos"], st["left"] = tok, st["pos"] + 1, st["left"] - 1
                if st["left"] <= 0:
                    r = st["req"]
                    recs.append(dict(id=r["id"], ttft_s=st["t_first"] - r["t"], t_seen=st["t_seen"], t_first=st["t_first"], n_out=r["n_out"]))
                    store.set(f"free/{drank}/{r['slot']}/{r['gen']}", "1")
                    del active[s]
        result = {"role": "decode", "requests": recs, "decode_tok_s_busy": tokens / max(t_busy, 1e-9), "tokens": tokens,
                  "unfinished": len(pending) + len(active), "status": eng.check_status()}

    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        pre = [x for g in gathered if g["role"] == "prefill" for x in g["requests"]]
        dec = [x for g in gathered if g["role"] == "decode" for x in g["requests"]]
        ft = [x["flow_time_ms"] for x in pre]
        dev_ms = [x["transfer_device_ms"] for x in pre]
        ttft = [x["ttft_s"] for x in dec]
        summary = {
            "arm": a.arm, "requests": len(reqs), "prefilled": len(pre), "decoded": len(dec),
            "kv_transfer_flow_time_ms_p50": ctl.percentile(ft, 0.5), "kv_transfer_flow_time_ms_p99": ctl.percentile(ft, 0.99),
            "kv_transfer_device_ms_p50": ctl.percentile(dev_ms, 0.5), "kv_transfer_device_ms_p99": ctl.percentile(dev_ms, 0.99),
            "kv_transfer_gbs_mean": sum(x["gbs"] for x in pre) / max(1, len(pre)),
            "ttft_s_mean": sum(ttft) / max(1, len(ttft)), "ttft_s_p50": ctl.percentile(ttft, 0.5),
            "decode_tok_s_busy_sum": sum(g["decode_tok_s_busy"] for g in gathered if g["role"] == "decode"),
            "offload_gb_s_per_prefill_gpu": [g["offload_gb_s"] for g in gathered if g["role"] == "prefill"],
            "unfinished": sum(g.get("unfinished", 0) for g in gathered if g["role"] == "decode"),
        }
        out = {"env": env_info(), "config": vars(a), "summary": summary, "prefill_records": pre, "decode_records": dec}
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        json.dump(out, open(a.out, "w"), indent=1)
        print(json.dumps(summary, indent=1))
    dist.barrier()
    if daemon is not None:
        daemon.stop()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
