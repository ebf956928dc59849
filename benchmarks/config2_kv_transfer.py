"""Point-to-point KV transfer between GPUs: Qwen3-8B-shaped paged KV (36 layers x 8 KV heads x 128, bf16, 16-token
blocks, randomly permuted block tables, N(0,1) values), sequence lengths uniform 1k-64k.

    python benchmarks/config2_kv_transfer.py [--gpus 2] [--requests 12] [--out results/config2.json] [--ref]

One process drives all GPUs (peer access). Arms:
  kernel        this runtime's paged gather + layout + peer-store kernel, unpaced
  kernel@X%     the same under a byte budget of X % of the unpaced rate (in-kernel credit gate, 1 ms grant windows)
  memcpy_peer   the reference's mechanism: one contiguous cudaMemcpyPeerAsync per request (no block table, no layout change)
  per_page      one peer copy per block: what a copy-engine design pays for a paged cache
  pairs         GPU 2i -> 2i+1 for all pairs at once (aggregate GB/s)
  fanout        GPU0 -> k destinations in one launch (replicated stores), and the same through an NVLink multicast
                address (multimem.st: the payload leaves GPU0 once)
  --ref         also runs the reference's own kv_nvlink_transfer_trace binary (baseline/_ref/bin) with the same geometry
Every time is a device time: CUDA events on the source stream, and the kernel's own globaltimer stamps.
Roofline: payload bytes over NVLink at 900 GB/s per direction (nominal) and 770 GB/s (measured peer copy).
"""
import argparse
import json
import os
import re
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from skygdr_b200 import ops  # noqa: E402
from skygdr_b200._ext import load  # noqa: E402
from skygdr_b200.cli.common import ResultFile, env_info  # noqa: E402

NVLINK_NOMINAL, NVLINK_MEASURED = 900.0, 770.0


def make_pair(src_gpu, dst_gpus, geom, max_blocks, seed):
    C = load()
    for d in dst_gpus:
        if d != src_gpu:
            assert C.enable_peer_access(src_gpu, d) and C.enable_peer_access(d, src_gpu)
    sdev = torch.device("cuda", src_gpu)
    src = ops.PagedKVPool(geom, max_blocks, "nhd", device=sdev)
    for i in range(0, max_blocks, 256):
        src.data[i:i + 256].normal_()
    dsts = [ops.PagedKVPool(geom, max_blocks, "hnd", device=torch.device("cuda", d)) for d in dst_gpus]
    g = torch.Generator().manual_seed(seed)
    sp = torch.randperm(max_blocks, generator=g).int().to(sdev)
    dp = torch.randperm(max_blocks, generator=g).int().to(sdev)
    return src, dsts, sp, dp


def time_kernel(flow, src, remotes, sp, dp, blocks_list, replicate=False, paced=False):
    """Returns (bytes, seconds by events, seconds by in-kernel timers, stall_ns)."""
    dev = src.data.device
    tot_b, tot_ev, tot_k, stall = 0, 0.0, 0.0, 0
    for nb in blocks_list:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.device(dev):
            e0.record()
            if paced:
                st = flow.transfer_to_completion(src, remotes, sp[:nb], dp[:nb], replicate=replicate)
            else:
                flow.transfer(src, remotes, sp[:nb], dp[:nb], replicate=replicate)
                st = flow.result()
            e1.record()
            e1.synchronize()
        assert st["status"] == 0, st
        tot_b += st["bytes_done"]
        tot_ev += e0.elapsed_time(e1) * 1e-3
        tot_k += st["device_time_ms"] * 1e-3
        stall += st["stall_ns"]
    return tot_b, tot_ev, tot_k, stall


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=min(2, torch.cuda.device_count()))
    ap.add_argument("--requests", type=int, default=12)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default="results/config2.json")
    ap.add_argument("--ref", action="store_true")
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--pages-per-chunk", type=int, default=8)
    ap.add_argument("--skip", default="", help="comma list of arm groups to leave out: paced, copy_engine, pairs, fanout, multimem")
    ap.add_argument("--resume", action="store_true", help="keep the arms that --out already holds and measure only the missing ones")
    a = ap.parse_args()
    skip = set(filter(None, a.skip.split(",")))
    assert a.gpus >= 2, "needs at least two GPUs"
    geom = ops.KVGeometry()
    g = torch.Generator().manual_seed(a.seed)
    seq = torch.randint(1024, 65536 + 1, (a.requests,), generator=g).tolist()
    blocks = [geom.blocks_for(t) for t in seq]
    max_blocks = max(blocks)
    rf = ResultFile(a.out, {"config": {"geometry": "36 layers x 8 kv heads x 128, bf16, 16-token blocks", "seq_lens": seq,
                                       "total_gb": sum(blocks) * geom.block_elems * 2 / 1e9, "gpus": a.gpus}, "env": env_info()}, resume=a.resume)
    res = rf.data                                  # every finished arm is written to --out at once (rf.save / rf.put)
    src, dsts, sp, dp = make_pair(0, [1], geom, max_blocks, a.seed)
    remotes = [ops.RemotePool.of(dsts[0])]
    flow = ops.KvTransferFlow("cuda:0", ctas=a.ctas or None, pages_per_chunk=a.pages_per_chunk)
    time_kernel(flow, src, remotes, sp, dp, blocks[:2])                      # warm-up
    b, ev, k, _ = time_kernel(flow, src, remotes, sp, dp, blocks)
    unpaced = b / k / 1e9
    res["arms"]["kernel"] = {"gb": b / 1e9, "gbs_events": b / ev / 1e9, "gbs_kernel_timer": unpaced, "frac_of_900": unpaced / NVLINK_NOMINAL,
                             "frac_of_measured_770": unpaced / NVLINK_MEASURED}
    # correctness of the last request, bit-exact
    nb = blocks[-1]
    ok = torch.equal(dsts[0].data[dp[:nb].long().to(dsts[0].data.device)], ops.reference_transfer(src, sp[:nb]).to(dsts[0].data.device))
    res["arms"]["kernel"]["exact"] = bool(ok)
    rf.save()
    # paced arms
    for pct in (() if "paced" in skip else (75, 50, 25)):
        if rf.done(f"kernel@{pct}%"):
            continue
        page = ops.CreditPage(flow_id=pct, unlimited=False)
        pf = ops.KvTransferFlow("cuda:0", page=page, ctas=a.ctas or None, pages_per_chunk=a.pages_per_chunk, max_wait_ms=20.0)
        budget = unpaced * pct / 100.0
        pacer = ops.LocalPacer(page, budget, window_ms=1.0).start(base=0)
        t0 = time.perf_counter()
        b, ev, k, stall = time_kernel(pf, src, remotes, sp, dp, blocks[: max(4, a.requests // 2)], paced=True)
        wall = time.perf_counter() - t0
        pacer.stop()
        rf.put(f"kernel@{pct}%", {"budget_gbs": budget, "achieved_gbs": b / ev / 1e9, "achieved_over_budget": b / ev / 1e9 / budget,
                                  "stall_ms_per_cta_sum": stall * 1e-6, "wall_s": wall})
    # baselines through the copy engine
    sdev, ddev = src.data.device, dsts[0].data.device
    for name in (() if "copy_engine" in skip else ("memcpy_peer", "per_page")):
        if rf.done(name):
            continue
        tot_b, tot_s = 0, 0.0
        for i, nb in enumerate(blocks):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.device(sdev):
                e0.record()
                if name == "memcpy_peer":
                    dsts[0].data[:nb].view(-1).copy_(src.data[:nb].view(-1), non_blocking=True)
                else:
                    spl, dpl = sp[:nb].tolist(), dp[:nb].tolist()
                    for x, y in zip(spl, dpl):
                        dsts[0].data[y].view(-1).copy_(src.data[x].view(-1), non_blocking=True)
                e1.record()
                e1.synchronize()
            if i >= 1:                                                       # first one warms up
                tot_b += nb * geom.block_elems * 2
                tot_s += e0.elapsed_time(e1) * 1e-3
        rf.put(name, {"gbs": tot_b / tot_s / 1e9, "frac_of_900": tot_b / tot_s / 1e9 / NVLINK_NOMINAL})
    del src, dsts
    torch.cuda.empty_cache()
    # all pairs at once
    if a.gpus >= 4 and "pairs" not in skip and not rf.done(f"pairs_x{a.gpus // 2}"):
        pairs = [(2 * i, 2 * i + 1) for i in range(a.gpus // 2)]
        sets = [make_pair(s, [d], geom, max_blocks, a.seed + s) for s, d in pairs]
        flows = [ops.KvTransferFlow(f"cuda:{s}") for s, _ in pairs]
        nb = blocks[0]
        for rep in range(3):
            for (src_p, dd, sp_p, dp_p), fl in zip(sets, flows):
                with torch.cuda.device(src_p.data.device):
                    fl.transfer(src_p, [ops.RemotePool.of(dd[0])], sp_p[:nb], dp_p[:nb])
            sts = [fl.result() for fl in flows]
        t_max = max(st["device_time_ms"] for st in sts) * 1e-3
        t0 = min(st["t_start_ns"] for st in sts)
        rf.put(f"pairs_x{len(pairs)}", {"aggregate_gbs_max_over_pairs": sum(st["bytes_done"] for st in sts) / t_max / 1e9,
                                        "per_pair_gbs": [st["bytes_done"] / (st["device_time_ms"] * 1e-3) / 1e9 for st in sts]})
        del sets
        torch.cuda.empty_cache()
    # fan-out from GPU0
    for k in sorted({min(a.gpus - 1, x) for x in (2, 4, 7)}):
        if k < 2 or "fanout" in skip or (rf.done(f"fanout_x{k}") and rf.done(f"fanout_multimem_x{k}")):
            continue
        src, dsts, sp, dp = make_pair(0, list(range(1, k + 1)), geom, min(max_blocks, 1024), a.seed)
        fl = ops.KvTransferFlow("cuda:0")
        nb = min(blocks[0], 1024)
        rem = [ops.RemotePool.of(d) for d in dsts]
        fl.transfer(src, rem, sp[:nb], dp[:nb], replicate=True); fl.result()
        fl.transfer(src, rem, sp[:nb], dp[:nb], replicate=True)
        st = fl.result()
        ok = all(torch.equal(d.data[dp[:nb].long().to(d.data.device)], ops.reference_transfer(src, sp[:nb]).to(d.data.device)) for d in dsts)
        res["arms"][f"fanout_x{k}"] = {"egress_gbs": st["bytes_done"] / (st["device_time_ms"] * 1e-3) / 1e9, "frac_of_900": st["bytes_done"] / (st["device_time_ms"] * 1e-3) / 1e9 / 900.0, "exact": bool(ok)}
        # the same fan-out through an NVLink multicast address: the payload leaves GPU0 once, NVSwitch replicates it
        try:
            if "multimem" in skip:
                raise RuntimeError("left out by --skip multimem")
            team = [0] + list(range(1, k + 1))
            with ops.MulticastPools(geom, min(max_blocks, 1024), team) as mc:
                for pool in mc.pools:
                    pool.data.zero_()
                for d in team:
                    torch.cuda.synchronize(d)
                flags = [ops.RemotePool(0, mc.pools[0].strides, geom.kv_heads) for _ in range(k)]   # no done flags; k destinations
                fl2 = ops.KvTransferFlow("cuda:0", method="simt")
                fl2.transfer(src, flags, sp[:nb], dp[:nb], replicate=True, multicast_ptr=mc.multicast_ptr); fl2.result()
                fl2.transfer(src, flags, sp[:nb], dp[:nb], replicate=True, multicast_ptr=mc.multicast_ptr)
                st = fl2.result()
                want = ops.reference_transfer(src, sp[:nb])
                ok = st["status"] == 0 and all(torch.equal(pl.data[dp[:nb].long().to(pl.data.device)], want.to(pl.data.device)) for pl in mc.pools[1:])
                sec = st["device_time_ms"] * 1e-3
                res["arms"][f"fanout_multimem_x{k}"] = {"egress_gbs": st["bytes_done"] / sec / 1e9, "delivered_gbs": k * st["bytes_done"] / sec / 1e9,
                                                        "frac_of_900_per_destination": st["bytes_done"] / sec / 1e9 / 900.0, "exact": bool(ok),
                                                        "granularity": int(mc.region.granularity)}
                del want
        except Exception as exc:                                             # no multicast support on this machine: say so, keep the unicast arm
            res["arms"][f"fanout_multimem_x{k}"] = {"unavailable": repr(exc)[:300]}
        rf.save()
        del src, dsts
        torch.cuda.empty_cache()
    if a.ref:
        exe = os.path.join(ROOT, "baseline", "_ref", "bin", "kv_nvlink_transfer_trace")
        if os.path.exists(exe):
            r = subprocess.run([exe, "--src", "0", "--dst", "1", "--iters", "200", "--dist", "computed", "--layers", "36", "--kv-heads", "8", "--head-dim", "128",
                                "--elem-bytes", "2", "--max-tokens", "65536", "--seed", "1"], capture_output=True, text=True, timeout=600)
            m = re.search(r"bw:\s+([0-9.]+) GiB/s", r.stdout)
            res["arms"]["reference_binary_trace"] = {"gib_s": float(m.group(1)) if m else None, "gbs": float(m.group(1)) * 1.073741824 if m else None,
                                                     "rc": r.returncode, "tail": r.stdout.strip().splitlines()[-6:]}
            exe2 = os.path.join(ROOT, "baseline", "_ref", "bin", "kv_nvlink_transfer")
            r = subprocess.run([exe2, "0", "1", "4096", "50"], capture_output=True, text=True, timeout=600)
            m = re.search(r"=\s*([0-9.]+) GiB/s", r.stdout)
            res["arms"]["reference_binary_fixed_4GiB"] = {"gib_s": float(m.group(1)) if m else None, "gbs": float(m.group(1)) * 1.073741824 if m else None, "rc": r.returncode}
        else:
            res["arms"]["reference_binary_trace"] = {"unavailable": "baseline/_ref/bin not built (run baseline/build_ref.sh)"}
    rf.save()
    print(json.dumps(res["arms"], indent=1))


if __name__ == "__main__":
    main()
