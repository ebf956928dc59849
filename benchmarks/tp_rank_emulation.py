"""One rank's share of a tensor-parallel decode step on one GPU, in three forms, to tell compute from communication.

    python benchmarks/tp_rank_emulation.py --tp 8 [--steps 8] [--layers 36] [--collective oneshot|rs_ag]

A model whose widths are 1 / tp of Qwen3-8B (heads, FFN, vocabulary) at the full hidden size, with the batch of a
tp-way run (16 x tp sequences, context 2k-16k): kernel shapes, launch counts and bytes per GPU are those of one rank at
TP = tp. Three engines step it, each as a CUDA graph, device-timed with CUDA events:

    tensor_parallel_engine   parallel.TPDecoder with world size 1: the collectives degenerate to this GPU pushing to itself,
                             so every fence, arrival counter and wait of the real step is there, the NVLink crossing is not.
                             A real tp-GPU step minus this is what crossing NVLink and waiting for peers costs.
    single_gpu_engine        models.Qwen3Decoder on the same shapes: this package's GEMMs and small kernels, no collective code
                             at all. tensor_parallel_engine minus this is what the collective's device-side protocol costs.
    library_arm              parallel.NcclTPDecoder with one rank: torch.matmul (cuBLAS) GEMMs, no collective. single_gpu_engine
                             minus this is the GEMM difference at these shapes.

It also prints an eager per-kernel-kind profile of the tensor-parallel engine (one CUDA event after every kernel; read it
for shares, eager launches add host gaps).
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from skygdr_b200.models import Qwen3Config  # noqa: E402
from skygdr_b200.models.qwen3 import Qwen3Decoder, Qwen3Weights  # noqa: E402
from skygdr_b200.ops.kv_cache import KVGeometry, PagedKVPool  # noqa: E402
from skygdr_b200.parallel.nccl_baseline import NcclTPDecoder  # noqa: E402
from skygdr_b200.parallel.tp import TPDecoder  # noqa: E402


def time_graph(engine, steps):
    for _ in range(3):
        engine.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        engine.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--attn-chunk", type=int, default=1024)
    ap.add_argument("--collective", default="oneshot", choices=["oneshot", "rs_ag"])
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    full = Qwen3Config()
    vs = (full.vocab + a.tp - 1) // a.tp
    cfg = Qwen3Config(layers=a.layers, q_heads=full.q_heads // a.tp, kv_heads=full.kv_heads // a.tp, ffn=full.ffn // a.tp, vocab=vs,
                      name=f"qwen3-8b/tp{a.tp}-rank")
    batch = 16 * a.tp
    g = torch.Generator().manual_seed(0)
    ctx = torch.randint(2048, 16384 + 1, (batch,), generator=g)
    extra = 16 * a.steps + 64
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
    ids0 = torch.zeros(batch, dtype=torch.int32, device=dev)
    eng = TPDecoder(cfg, w, pool, batch, max_ctx, 0, 1, a.attn_chunk, collective=a.collective)
    eng.set_batch(ids0, ctx.int().to(dev), table.to(dev))
    eng.profile_step(max_ctx)
    prof = eng.profile_step(max_ctx)
    eng.capture(batch, max_ctx)
    out = {"tp": a.tp, "batch": batch, "layers": a.layers, "collective": a.collective, "ms_per_step": {}}
    lib = NcclTPDecoder.from_engine(eng, collective="allreduce")
    lib.capture(batch, max_ctx)
    out["ms_per_step"]["library_arm"] = time_graph(lib, a.steps)
    del lib
    single = Qwen3Decoder(cfg, w, pool, batch, max_ctx, a.attn_chunk, "tc")
    single.set_batch(ids0, ctx.int().to(dev), table.to(dev))
    single.capture(batch, max_ctx)
    out["ms_per_step"]["single_gpu_engine"] = time_graph(single, a.steps)
    out["single_gpu_engine_status"] = single.check_status()
    del single
    out["ms_per_step"]["tensor_parallel_engine"] = time_graph(eng, a.steps)
    out["tensor_parallel_engine_status"] = eng.check_status()
    out["eager_profile_ms"] = prof
    out["bytes_per_step"] = eng.bytes_per_step(ctx)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
