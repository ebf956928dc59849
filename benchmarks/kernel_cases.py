"""Small, self-contained cases of each kernel, for timing and for profiler captures.

    python benchmarks/kernel_cases.py attn   [--batch 16 --ctx 8192 --kv-heads 8 --q-heads 32 --chunk 1024]
    python benchmarks/kernel_cases.py pattn  [--ctx 16384 --batch 1 --impl tc|sdpa]     (causal prefill attention over the paged pool)
    python benchmarks/kernel_cases.py gemm   [--m 16 --n 12288 --k 4096 --gated --splits 0]
    python benchmarks/kernel_cases.py kvt    [--blocks 256]         (same-GPU destination)
    python benchmarks/kernel_cases.py memhog [--gb 2 --op axpy]
    python benchmarks/kernel_cases.py norm   [--rows 16]

Each case holds well under a few GB, touches more than the 126 MB L2 per launch where the kernel is
bandwidth-bound, runs `--iters` launches after `--warm` warm-ups, and prints one JSON line with the
CUDA-event time per launch and the achieved fraction of the measured peaks (MEASURED_PEAKS.json,
fallback 6650 GB/s and 1590 TFLOP/s).
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import skygdr_b200.ops as ops  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


REPS = 1


def timed(fn, warm, iters, flush):
    """Median and best time of one call of fn in ms. With --reps R > 1 an event pair brackets R back-to-back calls (for inputs
    larger than L2, with --no-flush): the first call absorbs the host's launch latency, which otherwise sits inside the interval
    of a kernel that is shorter than the Python path that launches it."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(REPS):
            fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) / REPS)
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["attn", "pattn", "gemm", "kvt", "memhog", "norm"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warm", type=int, default=2)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--chunk", type=int, default=1024)
    ap.add_argument("--m", type=int, default=16)
    ap.add_argument("--n", type=int, default=12288)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--gated", action="store_true")
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--ntok", type=int, default=0, help="gemm: token tile (0 = chosen by the package)")
    ap.add_argument("--tile", default="", choices=["", "wide", "narrow"], help="gemm with more than 256 tokens: 256 x 256 or 128 x 256 tiles (default: chosen by the package)")
    ap.add_argument("--cluster", action="store_true", help="gemm with --splits: the K slices form a thread-block cluster and sum through distributed shared memory")
    ap.add_argument("--one-tile-per-cta", action="store_true", help="gemm with more than 256 tokens: the one-tile-per-CTA kernel instead of the persistent form")
    ap.add_argument("--blocks", type=int, default=256)
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--gb", type=float, default=2.0)
    ap.add_argument("--op", default="axpy")
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--reps", type=int, default=1, help="calls per event pair (see timed)")
    ap.add_argument("--impl", default="simt", choices=["simt", "tc", "sdpa"])
    a = ap.parse_args()
    global REPS
    REPS = max(1, a.reps)
    dev = "cuda"
    hbm, tf, src = peaks()
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = {"case": a.case, "peaks": src}
    if a.case == "pattn":
        # `--batch` prompts of `--ctx` tokens each; impl tc = this package's kernel on the pages in place,
        # sdpa = torch's scaled_dot_product_attention on contiguous K/V (the gather that feeds it is not timed)
        g = ops.KVGeometry(layers=1, kv_heads=a.kv_heads)
        n, B = a.ctx, a.batch
        nb = (n + 15) // 16
        pool = ops.PagedKVPool(g, B * nb + 1, "hnd")
        pool.data.normal_()
        table = (torch.randperm(B * nb, device=dev) + 1).int().view(B, nb)
        table = torch.cat([table, torch.zeros((B, 8), dtype=torch.int32, device=dev)], 1).contiguous()
        q = torch.randn((B * n, a.q_heads, 128), dtype=torch.bfloat16, device=dev)
        seq_start = (torch.arange(B + 1, device=dev) * n).int()
        flops = B * 2.0 * n * n * 128 * a.q_heads                  # causal: half of 4 n^2 d per head
        if a.impl == "sdpa":
            kv = pool.data[table[:, :nb].long().view(-1), 0].view(B, nb, 2, a.kv_heads, 16, 128)
            k = kv[:, :, 0].permute(0, 2, 1, 3, 4).reshape(B, a.kv_heads, nb * 16, 128)[:, :, :n].contiguous()
            v = kv[:, :, 1].permute(0, 2, 1, 3, 4).reshape(B, a.kv_heads, nb * 16, 128)[:, :, :n].contiguous()
            qs = q.view(B, n, a.q_heads, 128).transpose(1, 2).contiguous()
            fn = lambda: torch.nn.functional.scaled_dot_product_attention(qs, k, v, is_causal=True, enable_gqa=True)
            status = "library"
        else:
            attn = ops.PrefillAttention(dev)
            o_ = torch.empty_like(q)
            fn = lambda: attn(q, pool, 0, table, seq_start, n, out=o_)
        ms, best = timed(fn, a.warm, a.iters, flush)
        if a.impl != "sdpa":
            status = ops.read_status(attn.status)["status_name"]
        out.update(ms=ms, best_ms=best, flops=flops, tflops=flops / ms / 1e9, frac_bf16=flops / ms / 1e9 / tf, tokens=B * n, impl=a.impl, status=status)
    elif a.case == "attn":
        g = ops.KVGeometry(layers=1, kv_heads=a.kv_heads)
        gen = torch.Generator().manual_seed(0)
        ctx = torch.randint(a.ctx // 2, a.ctx + 1, (a.batch,), generator=gen).int().to(dev)
        nblk = int(((ctx + 15) // 16).sum()) + 1
        pool = ops.PagedKVPool(g, nblk, "hnd")
        pool.data.normal_()
        mb = (int(ctx.max()) + 15) // 16
        table = torch.zeros((a.batch, mb), dtype=torch.int32, device=dev)
        perm = torch.randperm(nblk, device=dev).int()
        o = 0
        for b in range(a.batch):
            nb = (int(ctx[b]) + 15) // 16
            table[b, :nb] = perm[o:o + nb]
            o += nb
        q = torch.randn((a.batch, a.q_heads, 128), dtype=torch.bfloat16, device=dev)
        attn = ops.PagedAttention(dev, a.batch, a.q_heads, a.kv_heads, max_ctx=a.ctx, chunk_tokens=a.chunk, impl=a.impl)
        o_ = torch.empty_like(q)
        ms, best = timed(lambda: attn(q, pool, 0, table, ctx, max_ctx=int(ctx.max()), out=o_), a.warm, a.iters, flush)
        byt = int(ctx.sum()) * a.kv_heads * 128 * 2 * 2
        out.update(ms=ms, best_ms=best, kv_bytes=byt, gbs=byt / ms / 1e6, frac_hbm=byt / ms / 1e6 / hbm, tokens=int(ctx.sum()), impl=a.impl,
                   status=ops.read_status(attn.status)["status_name"])
        if a.impl == "tc":
            from skygdr_b200._ext import load
            out["one_tma_request_per_page"] = bool(load().paged_attn_tc_page_box() == 1)
    elif a.case == "gemm":
        x = torch.randn((a.m, a.k), dtype=torch.bfloat16, device=dev)
        w = torch.randn((a.n * (2 if a.gated else 1), a.k), dtype=torch.bfloat16, device=dev) / 64
        y = torch.empty((a.m, a.n), dtype=torch.bfloat16, device=dev)
        ms, best = timed(lambda: ops.gemm(x, w, out=y, gated=a.gated, splits=a.splits or None, ntok=a.ntok, persistent=False if a.one_tile_per_cta else (a.tile or None), cluster=a.cluster),
                         a.warm, a.iters, flush)
        from skygdr_b200.ops.gemm import workspace_for

        out["status"] = ops.read_status(workspace_for(dev).status)["status_name"]
        out["form"] = ("one tile per CTA" + (", split-K inside a cluster" if a.cluster else "")) if (a.one_tile_per_cta or a.m <= 256) else "persistent, " + (a.tile or "tile chosen by the package")
        byt = (w.numel() + x.numel() + y.numel()) * 2
        fl = 2.0 * a.m * w.shape[0] * a.k
        out.update(ms=ms, best_ms=best, bytes=byt, gbs=byt / ms / 1e6, frac_hbm=byt / ms / 1e6 / hbm, tflops=fl / ms / 1e9,
                   frac_tensor=fl / ms / 1e9 / tf, splits=a.splits or ops.pick_splits(a.m, a.n, a.k, 148, a.gated))
    elif a.case == "kvt":
        g = ops.KVGeometry()
        src_p = ops.PagedKVPool(g, a.blocks, "nhd")
        src_p.data.normal_()
        dst_p = ops.PagedKVPool(g, a.blocks, "hnd")
        sb = torch.randperm(a.blocks, device=dev).int()
        db = torch.randperm(a.blocks, device=dev).int()
        flow = ops.KvTransferFlow(dev, ctas=a.ctas or None)
        ms, best = timed(lambda: flow.transfer(src_p, [ops.RemotePool.of(dst_p)], sb, db), a.warm, a.iters, None)
        byt = ops.link_bytes(g, a.blocks)
        out.update(ms=ms, best_ms=best, payload_bytes=byt, gbs=byt / ms / 1e6, hbm_traffic_frac=2 * byt / ms / 1e6 / hbm)
    elif a.case == "memhog":
        hog = ops.Memhog(dev, gb=a.gb, op=a.op, ctas=a.ctas or None)
        hog.launch(iters=1)
        hog.result()
        hog.launch(iters=a.iters)
        r = hog.result()
        out.update(seconds=r["seconds"], gbs=r["gb_s"], frac_hbm=r["gb_s"] / hbm, bytes=r["bytes_done"])
    else:
        x = torch.randn((a.rows, 4096), dtype=torch.bfloat16, device=dev)
        res = torch.randn_like(x)
        w = torch.ones(4096, dtype=torch.bfloat16, device=dev)
        y = torch.empty_like(x)
        ms, best = timed(lambda: ops.rmsnorm(x, w, 1e-6, residual=res, out=y), a.warm, a.iters, None)
        out.update(ms=ms, best_ms=best)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
