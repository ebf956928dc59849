"""What SM-originated stores into a peer GPU's memory can reach on this machine, beside the copy engine and beside the
paged transfer kernel: the ceiling that `kv_transfer` is measured against.

    python benchmarks/peer_store_ceiling.py [--src 0 --dst 1] [--gb 2] [--iters 3] [--out results/peer_store_ceiling.json]
    python benchmarks/peer_store_ceiling.py --multicast 0,1,2 ...      (also: multimem.st through one multicast address)

One process, two (or more) GPUs. Arms, all writing `--gb` of the destination per round, device-timed with CUDA events:
  memcpy_peer         cudaMemcpyPeerAsync, contiguous (the copy engine: the reference's mechanism,
                      llm_problem_analysis/kv_nvlink_transfer.cu:109-137)
  st.v4               st.global.v4 from registers, no loads (csrc/kernels/peer_store_probe.cu mode 0), 148-1184 CTAs
  bulk <S> x <G>      cp.async.bulk shared -> global of S bytes with G groups outstanding per CTA (mode 1), 148 / 296 CTAs
  multimem.st         the register store through the NVLink multicast address (mode 2): egress counted once
  kv_transfer         the paged transfer kernel itself on the same pair (gather + NHD -> HND + peer stores)
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from skygdr_b200 import ops  # noqa: E402
from skygdr_b200._ext import load  # noqa: E402
from skygdr_b200.cli.common import env_info  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", type=int, default=0)
    ap.add_argument("--dst", type=int, default=1)
    ap.add_argument("--gb", type=float, default=2.0)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--multicast", default="", help="comma-separated team of GPUs (first = source) for the multimem.st arm")
    ap.add_argument("--out", default="results/peer_store_ceiling.json")
    a = ap.parse_args()
    C = load()
    assert C.enable_peer_access(a.src, a.dst), "no peer access"
    nbytes = int(a.gb * 1e9) // (1 << 20) * (1 << 20)
    dst = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{a.dst}")
    srcbuf = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{a.src}")
    torch.cuda.set_device(a.src)
    rows = []

    def best(fn, n=a.iters):
        fn()
        return min(fn() for _ in range(n))

    # copy engine
    def memcpy():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dst.copy_(srcbuf, non_blocking=True)
        e1.record()
        torch.cuda.synchronize(a.src)
        return e0.elapsed_time(e1)

    ms = best(memcpy)
    rows.append({"arm": "memcpy_peer (copy engine)", "ms": ms, "gbs": nbytes / ms / 1e6})
    for ctas in (148, 296, 592, 1184):
        ms = best(lambda: C.peer_store_probe(a.src, dst.data_ptr(), nbytes, 0, ctas=ctas))
        rows.append({"arm": "st.v4", "ctas": ctas, "ms": ms, "gbs": nbytes // ctas // 4096 * 4096 * ctas / ms / 1e6})
    for ctas in (148, 296):
        for sb in (4096, 16384, 32768, 65536):
            for infl in (1, 2, 4, 8):
                ms = best(lambda: C.peer_store_probe(a.src, dst.data_ptr(), nbytes, 1, store_bytes=sb, inflight=infl, ctas=ctas))
                rows.append({"arm": f"bulk {sb // 1024}K x {infl}", "ctas": ctas, "ms": ms, "gbs": nbytes // ctas // sb * sb * ctas / ms / 1e6})
    # the transfer kernel on the same pair
    geom = ops.KVGeometry()
    nb = max(64, nbytes // (geom.block_elems * 2))
    spool = ops.PagedKVPool(geom, nb, "nhd", device=f"cuda:{a.src}")
    dpool = ops.PagedKVPool(geom, nb, "hnd", device=f"cuda:{a.dst}")
    sb_ = torch.randperm(nb, device=f"cuda:{a.src}").int()
    db_ = torch.randperm(nb, device=f"cuda:{a.src}").int()
    flow = ops.KvTransferFlow(f"cuda:{a.src}")
    for _ in range(2):
        flow.transfer(spool, [ops.RemotePool.of(dpool)], sb_, db_)
        st = flow.result()
    rows.append({"arm": "kv_transfer (paged gather + layout change + peer stores)", "ms": st["device_time_ms"],
                 "gbs": st["bytes_done"] / st["device_time_ms"] / 1e6, "status": st["status"]})
    del spool, dpool
    if a.multicast:
        team = [int(x) for x in a.multicast.split(",")]
        ok, why = C.multicast_supported(team[0])
        if ok:
            region = C.multicast_create(team, nbytes)
            try:
                for ctas in (148, 296, 592, 1184):
                    ms = best(lambda: C.peer_store_probe(team[0], int(region.multicast), nbytes, 2, ctas=ctas))
                    rows.append({"arm": f"multimem.st to {len(team)} GPUs", "ctas": ctas, "ms": ms, "egress_gbs": nbytes // ctas // 4096 * 4096 * ctas / ms / 1e6})
            finally:
                C.multicast_destroy(region)
        else:
            rows.append({"arm": "multimem.st", "skipped": why})
    out = {"env": env_info(), "bytes_per_round": nbytes, "src": a.src, "dst": a.dst, "rows": rows}
    os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
    json.dump(out, open(a.out, "w"), indent=1)
    for r in rows:
        print(json.dumps(r))
    sm = [r for r in rows if r["arm"].startswith(("st.v4", "bulk"))]
    print("best SM-originated store:", json.dumps(max(sm, key=lambda r: r["gbs"])))


if __name__ == "__main__":
    main()
