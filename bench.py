"""Headline benchmark: Qwen3-8B decode throughput with tensor parallelism over N GPUs.

    python bench.py --gpus 1 --steps 32 --warmup 4
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...

Workload: random-init Qwen3-8B (36 layers, hidden 4096, 32/8 heads of 128, FFN 12288, vocabulary
151936), bf16, paged KV cache with 16-token blocks and randomly permuted block tables filled with
N(0,1) values, context lengths uniform in [2k, 16k] (seed 0), greedy sampling. Global batch is
16 x N (batch 128 at TP=8): weights and KV heads are sharded N ways, so the KV bytes per GPU stay
fixed as N grows ("weak" scaling); a batch-128 cache at 2k-16k context (about 170 GB) does not fit
one GPU next to the weights.

One timed step = embedding, 36 decoder layers (RMSNorm, QKV GEMM, QK-norm + RoPE + KV append, paged
GQA attention, O GEMM, RMSNorm, gated gate/up GEMM, down GEMM, with the tensor-parallel
all-gather / reduce-scatter fused into those kernels), final norm, lm_head GEMM, argmax.
`value` times K CUDA-graph replays of that step with CUDA events (max over ranks); `e2e` times the
same K steps through `DecodeSession.step`, which also copies the step's token ids and positions from
pinned host memory and reads the sampled ids back.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch-per-gpu", type=int, default=16)
    ap.add_argument("--ctx-lo", type=int, default=2048)
    ap.add_argument("--ctx-hi", type=int, default=16384)
    ap.add_argument("--layers", type=int, default=36, help="for smoke runs only; the benchmark uses 36")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--attn-impl", default="tc", choices=["tc", "tcp", "simt"])
    ap.add_argument("--tp-collective", default="rs_ag", choices=["rs_ag", "oneshot"],
                    help="tensor-parallel form: reduce-scatter + all-gather (default) or the one-shot all-reduce")
    ap.add_argument("--attn-chunk", type=int, default=1024)
    ap.add_argument("--attn-order", default="seq", choices=["seq", "tail", "fine"],
                    help="tail: every sequence's partial last chunk is scheduled after all full chunks; fine: that part is also cut into "
                         "quarter chunks (neither has run on a GPU yet)")
    ap.add_argument("--fuse-norm", action="store_true",
                    help="1 GPU: RMSNorms folded into the GEMM epilogues, 6 kernels per layer instead of 8 (not yet run on a GPU)")
    ap.add_argument("--profile-step", action="store_true", help="also print per-kernel-kind times of one eager step (tensor-parallel engine)")
    return ap.parse_args()


def reference_arm(args) -> int:
    """The reference has no decoder model, no tensor parallelism and no Python package; see baseline/reference_arm.py."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra

    rank = int(os.environ.get("RANK", "0"))
    out = ra.run(args, rank)
    if rank == 0:
        print(json.dumps(out), flush=True)
    return 0


def main() -> int:
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(3, args.warmup)          # fewer than three warm-up steps would time first-use effects; the line reports what was done
    import torch
    import torch.distributed as dist

    from skygdr_b200.models import DecodeSession, Qwen3Config
    from skygdr_b200.parallel.tp import build_decode_engine
    from skygdr_b200.utils.clocks import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = Qwen3Config(layers=args.layers)
    batch = args.batch_per_gpu * world
    g = torch.Generator().manual_seed(args.seed)
    ctx = torch.randint(args.ctx_lo, args.ctx_hi + 1, (batch,), generator=g)
    total_steps = 2 * (args.steps + args.warmup) + 8
    max_ctx = int(ctx.max()) + total_steps + 1
    eng, table = build_decode_engine(cfg, dev, rank, world, ctx, total_steps, seed=args.seed, kv_init="normal",
                                     attn_chunk=args.attn_chunk, attn_impl=args.attn_impl, collective=args.tp_collective,
                                     fuse_norm=args.fuse_norm, attn_tail_order={"seq": False, "tail": True, "fine": "fine"}[args.attn_order])

    ids0 = torch.randint(0, cfg.vocab, (batch,), generator=g).int()
    eng.set_batch(ids0.to(dev), ctx.int().to(dev), table.to(dev))
    sess = DecodeSession(eng, batch, max_ctx)          # captures the step into a CUDA graph
    sess.start(ids0, ctx.int(), table)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-timed: K graph replays ----
    for _ in range(args.warmup):
        eng.replay()
    barrier()
    with ClockSampler(local) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            eng.replay()
        e1.record()
        barrier()
        dev_ms = e0.elapsed_time(e1)
        # ---- end to end through DecodeSession.step: H2D inputs, step, D2H result, every step ----
        sess.h_pos.copy_(eng.positions[:batch].cpu())
        sess.h_ids.copy_(eng.ids[:batch].cpu())
        for _ in range(args.warmup):
            sess.step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            sess.step()
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])
    status = eng.check_status()
    prof = None
    if args.profile_step and hasattr(eng, "profile_step"):
        eng.profile_step(max_ctx)
        prof = eng.profile_step(max_ctx)
        eng._advance(batch)

    if rank == 0:
        tok_s = batch * args.steps / (dev_ms * 1e-3)
        e2e_tok_s = batch * args.steps / (e2e_ms * 1e-3)
        hbm = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"] if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 6650.0
        step_bytes = eng.bytes_per_step(ctx + args.warmup + args.steps // 2)
        out = {
            "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random-init weights, N(0,1) KV, uniform context lengths)",
            "config": {"model": cfg.name if args.layers == 36 else f"{cfg.name}-{args.layers}L", "global_batch": batch,
                       "seq_len": f"context uniform {args.ctx_lo}-{args.ctx_hi}, 1 new token per step",
                       "parallelism": f"tp{world}", "kv_block_tokens": 16, "sampling": "greedy", "attention": f"{args.attn_impl}, {args.attn_chunk}-token splits" + ({"seq": "", "tail": ", partial chunks last", "fine": ", partial chunks last in quarter-chunk pieces"}[args.attn_order]),
                       "norms": "folded into the GEMM epilogues" if args.fuse_norm else "norm kernels",
                       "l2": "inputs larger than L2: each step streams %.1f GB of weights and KV per GPU" % (step_bytes / 1e9)},
            "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": sess.h2d_bytes_per_step, "d2h_bytes_per_step": sess.d2h_bytes_per_step},
            "gpu_launches": eng.kernels_per_step * args.steps,
            "clocks": clocks.summary(),
            "roofline": {"hbm_bytes_per_step_per_gpu": step_bytes, "hbm_gbs_achieved": step_bytes / (dev_ms / args.steps) / 1e6,
                         "hbm_frac_of_measured": step_bytes / (dev_ms / args.steps) / 1e6 / hbm},
            "kernel_status": status, "impl": "ours",
        }
        if prof:
            out["eager_step_profile_ms"] = prof
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
