"""kv_nvlink_transfer / kv_nvlink_transfer_trace: KV hand-off between two GPUs of one process.

    python -m skygdr_b200.cli.kv_nvlink_transfer <src_gpu=0> <dst_gpu=1> <size_mib=1024> <iters=100> [--method kernel|memcpy_peer|per_page]
    python -m skygdr_b200.cli.kv_nvlink_transfer --trace --src 0 --dst 1 --iters 200 --dist computed|cached|input --layers 36
           --kv-heads 8 --head-dim 128 --elem-bytes 2 --max-tokens 65536 --seed 1 [--method ...] [--budget-gbps G]

Positional form and the `KV transfer done:` line: llm_problem_analysis/kv_nvlink_transfer.cu:45-53,137. Trace form,
its flags and the `Trace-shaped KV transfer done:` block: llm_problem_analysis/kv_nvlink_transfer_trace.cu:49-71,404-408.

Methods: `kernel` (default) is this runtime's paged transfer kernel: gather by block table, token-major to
head-major, peer stores, credit gate. `memcpy_peer` is the reference's mechanism, one contiguous
cudaMemcpyPeerAsync per request; `per_page` is what a paged cache forces on a copy-engine design, one peer copy
per block. Both baselines are issued through torch (`Tensor.copy_` across devices).
Times are taken on the device (CUDA events on the source stream).
"""
from __future__ import annotations

import argparse
import sys
import time
from typing import List

GIB = float(1 << 30)


def run_transfers(src_gpu: int, dst_gpu: int, token_counts: List[int], geom, method: str, budget_gbps: float = 0.0, warmup: int = 4,
                  seed: int = 1):
    """Moves one request per entry of ``token_counts``; returns (total_bytes, device_seconds, per_request_ms)."""
    import torch

    from skygdr_b200 import ops
    from skygdr_b200._ext import load

    C = load()
    sdev, ddev = torch.device("cuda", src_gpu), torch.device("cuda", dst_gpu)
    if src_gpu != dst_gpu:
        assert C.enable_peer_access(src_gpu, dst_gpu) and C.enable_peer_access(dst_gpu, src_gpu), "no peer access between the GPUs"
    max_blocks = max(geom.blocks_for(t) for t in token_counts)
    torch.cuda.set_device(sdev)
    src = ops.PagedKVPool(geom, max_blocks, "nhd", device=sdev)
    for i in range(0, max_blocks, 256):
        src.data[i:i + 256].normal_()
    dst = ops.PagedKVPool(geom, max_blocks, "hnd", device=ddev)
    g = torch.Generator().manual_seed(seed)
    src_perm = torch.randperm(max_blocks, generator=g).int().to(sdev)
    dst_perm = torch.randperm(max_blocks, generator=g).int().to(sdev)
    page = pacer = None
    flow = ops.KvTransferFlow(sdev)
    if budget_gbps > 0:
        page = ops.CreditPage(flow_id=1, unlimited=False)
        flow = ops.KvTransferFlow(sdev, page=page, max_wait_ms=50.0)
    remote = ops.RemotePool.of(dst)
    stream = torch.cuda.Stream(sdev)

    def one(tokens: int):
        nb = geom.blocks_for(tokens)
        if method == "kernel":
            flow.transfer(src, [remote], src_perm[:nb], dst_perm[:nb])
        elif method == "memcpy_peer":
            dst.data[:nb].view(-1).copy_(src.data[:nb].view(-1), non_blocking=True)
        elif method == "per_page":
            sp, dp = src_perm[:nb].tolist(), dst_perm[:nb].tolist()
            for a, b in zip(sp, dp):
                dst.data[b].view(-1).copy_(src.data[a].view(-1), non_blocking=True)
        else:
            raise ValueError(method)
        return nb * geom.block_elems * 2

    per_ms, total = [], 0
    with torch.cuda.stream(stream):
        for t in token_counts[:warmup]:
            one(t)
            if method == "kernel":
                flow.result()
        torch.cuda.synchronize(sdev)
        if page is not None:
            pacer = ops.LocalPacer(page, budget_gbps, window_ms=1.0).start(base=flow.consumed)
        t_all0 = time.perf_counter()
        dev_s = 0.0
        for t in token_counts:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            total += one(t)
            if method == "kernel" and page is not None:
                st = flow.result()
                while st["status"] == 1:                 # yielded on credit: relaunch from the cursor
                    flow.resume(st)
                    st = flow.result()
            e1.record(stream)
            e1.synchronize()
            if method == "kernel" and page is None:
                flow.result()
            ms = e0.elapsed_time(e1)
            per_ms.append(ms)
            dev_s += ms * 1e-3
        wall = time.perf_counter() - t_all0
    if pacer:
        pacer.stop()
    return total, dev_s, per_ms, wall


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    ap = argparse.ArgumentParser()
    ap.add_argument("pos", nargs="*")
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--src", type=int, default=0)
    ap.add_argument("--dst", type=int, default=1)
    ap.add_argument("--iters", type=int, default=None)
    ap.add_argument("--dist", default="computed", choices=["input", "cached", "computed"])
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--elem-bytes", type=int, default=2)
    ap.add_argument("--max-tokens", type=int, default=65536)
    ap.add_argument("--sync-every", type=int, default=256)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--method", default="kernel", choices=["kernel", "memcpy_peer", "per_page"])
    ap.add_argument("--budget-gbps", type=float, default=0.0)
    a = ap.parse_args(argv)
    from skygdr_b200.control import ctl
    from skygdr_b200.ops import KVGeometry

    assert a.elem_bytes == 2 and a.head_dim == 128, "the transfer kernel moves bf16 pages of head_dim 128"
    geom = KVGeometry(a.layers, a.kv_heads, a.head_dim)
    def pct(v, q):                                        # the reference's index rule (kv_nvlink_transfer_trace.cu:255-266)
        v = sorted(v)
        return v[int(q * (len(v) - 1))] if v else 0

    if a.trace:
        iters = a.iters or 10000
        tokens = ctl.sample_trace_tokens(a.dist, a.seed, iters, a.max_tokens)
        dist = ctl.trace_dist(a.dist, a.max_tokens)
        nbytes = [geom.blocks_for(t) * geom.block_elems * 2 for t in tokens]
        # header block with the reference's labels (kv_nvlink_transfer_trace.cu:291-325), which its harnesses grep for
        print(f"src_gpu={a.src} dst_gpu={a.dst} iters={iters} dist={a.dist}")
        print("peer_access src->dst=1 dst->src=1")
        print(f"KV geometry: layers={a.layers} kv_heads={a.kv_heads} head_dim={a.head_dim} elem_bytes={a.elem_bytes}")
        print(f"Trace quantiles: p50={round(dist.inverse_cdf(0.5))} p90={round(dist.inverse_cdf(0.9))} p99={round(dist.inverse_cdf(0.99))} "
              f"max={round(dist.inverse_cdf(1.0))} tokens")
        print(f"sampled tokens: p50={pct(tokens, 0.5)} p90={pct(tokens, 0.9)} p99={pct(tokens, 0.99)} max={max(tokens)}")
        print(f"sampled bytes: p50={pct(nbytes, 0.5)} p90={pct(nbytes, 0.9)} p99={pct(nbytes, 0.99)} max={max(nbytes)}")
        print(f"max transfer allocation: {max(nbytes) / GIB:.2f} GiB (paged: whole 16-token blocks)", flush=True)
        total, dev_s, per_ms, wall = run_transfers(a.src, a.dst, tokens, geom, a.method, a.budget_gbps, seed=a.seed)
        gib = total / GIB
        print("Trace-shaped KV transfer done:")
        print(f"  transfers: {iters}")
        print(f"  total:     {gib:.2f} GiB")
        print(f"  time:      {dev_s:.3f} s")
        print(f"  bw:        {gib / dev_s:.2f} GiB/s")
        print(f"  bw_gb_s:   {total / dev_s / 1e9:.2f} GB/s   method={a.method} dist={a.dist} wall_s={wall:.3f}")
        print(f"  flow_time_ms p50={ctl.percentile(per_ms, 0.5):.3f} p99={ctl.percentile(per_ms, 0.99):.3f}")
        return 0
    src_gpu = int(a.pos[0]) if len(a.pos) > 0 else 0
    dst_gpu = int(a.pos[1]) if len(a.pos) > 1 else 1
    size_mib = int(a.pos[2]) if len(a.pos) > 2 else 1024
    iters = int(a.pos[3]) if len(a.pos) > 3 else (a.iters or 100)
    tokens_per = max(16, (size_mib << 20) // geom.bytes_per_token())
    print(f"src_gpu={src_gpu} dst_gpu={dst_gpu} size={size_mib} MiB iters={iters}", flush=True)
    total, dev_s, per_ms, wall = run_transfers(src_gpu, dst_gpu, [tokens_per] * iters, geom, a.method, a.budget_gbps, seed=a.seed)
    print(f"KV transfer done: {total / GIB:.2f} GiB in {dev_s:.3f} s = {total / GIB / dev_s:.2f} GiB/s ({total / dev_s / 1e9:.2f} GB/s) "
          f"method={a.method}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
