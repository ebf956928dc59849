"""One rank's share of a tensor-parallel decode step, on one GPU.

    python benchmarks/tp_rank_shapes.py --tp 8 [--steps 8] [--layers 36]

Runs the tensor-parallel engine with world size 1 on a model whose widths are 1/tp of Qwen3-8B (heads, FFN,
vocabulary) and the full hidden size, with the batch of a tp-way run (16 x tp). Kernel shapes, launch counts and
per-GPU bytes are those of one rank at TP=tp; the collectives degenerate to this GPU pushing to itself, so the
difference between this time and a real tp-GPU step is what crossing NVLink and waiting for peers costs.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from skygdr_b200.models import Qwen3Config  # noqa: E402
from skygdr_b200.parallel.tp import TPDecoder, build_decode_engine  # noqa: E402
from skygdr_b200.models.qwen3 import Qwen3Weights  # noqa: E402
from skygdr_b200.ops.kv_cache import KVGeometry, PagedKVPool  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--attn-chunk", type=int, default=1024)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    full = Qwen3Config()
    vs = (full.vocab + a.tp - 1) // a.tp
    cfg = Qwen3Config(layers=a.layers, q_heads=full.q_heads // a.tp, kv_heads=full.kv_heads // a.tp, ffn=full.ffn // a.tp, vocab=vs,
                      name=f"qwen3-8b/tp{a.tp}-rank")
    batch = 16 * a.tp
    g = torch.Generator().manual_seed(0)
    ctx = torch.randint(2048, 16384 + 1, (batch,), generator=g)
    extra = 4 * a.steps + 16
    w = Qwen3Weights(cfg, dev, seed=0)
    geom = KVGeometry(cfg.layers, cfg.kv_heads, 128)
    bps = [(int(c) + extra + 15) // 16 for c in ctx]
    pool = PagedKVPool(geom, sum(bps) + 1, "hnd", device=dev)
    max_ctx = int(ctx.max()) + extra + 1
    table = torch.zeros((batch, (max_ctx + 15) // 16), dtype=torch.int32)
    perm = (torch.randperm(sum(bps)) + 1).int()
    o = 0
    for i, nb in enumerate(bps):
        table[i, :nb] = perm[o:o + nb]
        o += nb
    eng = TPDecoder(cfg, w, pool, batch, max_ctx, 0, 1, a.attn_chunk)
    eng.set_batch(torch.zeros(batch, dtype=torch.int32, device=dev), ctx.int().to(dev), table.to(dev))
    eng.profile_step(max_ctx)
    prof = eng.profile_step(max_ctx)
    eng.capture(batch, max_ctx)
    for _ in range(3):
        eng.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        eng.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    print(json.dumps({"tp": a.tp, "batch": batch, "graph_ms_per_step": ms, "status": eng.check_status(), "eager_profile_ms": prof,
                      "bytes_per_step": eng.bytes_per_step(ctx)}))


if __name__ == "__main__":
    main()
