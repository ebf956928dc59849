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
GQA attention, O GEMM, RMSNorm, gated gate/up GEMM, down GEMM, with the tensor-parallel all-reduce
fused into those kernels: partial tiles pushed to the peers from the GEMM epilogue, summed by the
norm kernel), final norm, lm_head GEMM, argmax.
`value` times K CUDA-graph replays of that step with CUDA events (max over ranks); `e2e` times the
same K steps through `DecodeSession.step`, which also copies the step's token ids and positions from
pinned host memory and reads the sampled ids back.

`baseline` is the same decoder step built from library calls on the same GPUs, same weights and same
KV cache: torch.matmul (cuBLAS) for every GEMM and torch.distributed (NCCL) for the collectives, in
its two usual forms (all-reduce; reduce-scatter + all-gather), each captured in a CUDA graph like
ours; the faster form is the baseline and `vs_baseline` = value / that. `check` compares one step
of both engines from the same state (logits and sampled ids).
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
    ap.add_argument("--attn-impl", default="tc", choices=["tc", "simt"])
    ap.add_argument("--tp-collective", default="oneshot", choices=["oneshot", "rs_ag"],
                    help="tensor-parallel form: one-shot all-reduce (default) or reduce-scatter + all-gather")
    ap.add_argument("--attn-chunk", type=int, default=0, help="tokens per attention CTA; 0 = planned from the batch's context lengths")
    ap.add_argument("--no-baseline", action="store_true", help="skip the library (cuBLAS + NCCL) arm and the numeric check")
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
    from skygdr_b200.parallel.nccl_baseline import NcclTPDecoder
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
    n_arms = 1 if args.no_baseline else 3
    total_steps = (n_arms + 1) * (args.steps + args.warmup) + 16
    max_ctx = int(ctx.max()) + total_steps + 1
    eng, table = build_decode_engine(cfg, dev, rank, world, ctx, total_steps, seed=args.seed, kv_init="normal",
                                     attn_chunk=args.attn_chunk, attn_impl=args.attn_impl, collective=args.tp_collective)

    ids0 = torch.randint(0, cfg.vocab, (batch,), generator=g).int()
    eng.set_batch(ids0.to(dev), ctx.int().to(dev), table.to(dev))
    sess = DecodeSession(eng, batch, max_ctx)          # captures the step into a CUDA graph
    sess.start(ids0, ctx.int(), table)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(*vals):
        if world == 1:
            return vals
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return tuple(float(v) for v in t)

    def time_replays(engine) -> float:
        """K graph replays of `engine`, device-timed with CUDA events between two barriers; max over ranks, in ms."""
        for _ in range(args.warmup):
            engine.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            engine.replay()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))[0]

    with ClockSampler(local, period_s=0.01) as clocks:
        # ---- device-timed: K graph replays ----
        dev_ms = time_replays(eng)
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
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)[0]
    status = eng.check_status()

    # ---- the library arm on the same GPUs, weights and cache, and the numeric check against it ----
    baseline, check, baseline_error = None, None, None

    def library_arm_and_check():
        nonlocal baseline, check
        forms, libs = {}, {}
        for form in (("allreduce", "rs_ag") if world > 1 else ("allreduce",)):
            libs[form] = NcclTPDecoder.from_engine(eng, collective=form)
            libs[form].capture(batch, max_ctx)
            forms[form] = time_replays(libs[form])
        best = min(forms, key=forms.get)
        baseline = {"impl": "torch.matmul (cuBLAS) GEMMs" + (" + torch.distributed (NCCL) collectives" if world > 1 else "") +
                            "; attention, norms, RoPE and sampling are this package's kernels in both arms",
                    "form": best if world > 1 else "one GPU, no collective", "ms_per_step": forms[best] / args.steps,
                    "value": batch * args.steps / (forms[best] * 1e-3),
                    "all_forms_ms_per_step": {k: v / args.steps for k, v in forms.items()}}

        # One eager step of each engine from the same state: this rank's slice of the logits, and the sampled ids. Two correct
        # bf16 implementations of 36 layers differ by accumulated rounding; with more than one rank the two library forms
        # against each other give that floor.
        def logits_of(engine, state):
            engine.ids.copy_(state[0]); engine.positions.copy_(state[1]); engine.ctx_lens.copy_(state[2])
            engine.step(batch, max_ctx, advance=False)
            torch.cuda.synchronize(dev)
            return engine.logits[:batch].float().clone(), engine.next_ids[:batch].clone()

        def compare(a, b):
            d = a - b
            loc = torch.stack([d.pow(2).sum(), b.pow(2).sum()]).double()
            mx = torch.stack([d.abs().max(), b.abs().max()]).double()
            if world > 1:
                dist.all_reduce(loc)
                dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            return {"max_rel_err": float(mx[0] / mx[1].clamp_min(1e-30)), "rms_rel_err": float((loc[0] / loc[1].clamp_min(1e-30)).sqrt())}

        state = (eng.ids.clone(), eng.positions.clone(), eng.ctx_lens.clone())
        ours_logits, ours_ids = logits_of(eng, state)
        ref_logits, ref_ids = logits_of(libs["allreduce"], state)
        check = {"against": "library arm (all-reduce form), one eager step of all 36 layers from the same state; errors relative to the largest / rms logit",
                 **compare(ours_logits, ref_logits), "sampled_ids_equal": float((ours_ids == ref_ids).float().mean())}
        if "rs_ag" in libs:
            other_logits, other_ids = logits_of(libs["rs_ag"], state)
            check["library_forms_against_each_other"] = {**compare(other_logits, ref_logits),
                                                         "sampled_ids_equal": float((other_ids == ref_ids).float().mean())}
        # The floor at every N: the library arm with each GEMM summed in fp32 in another order (same bf16 rounding points).
        lib32 = NcclTPDecoder.from_engine(eng, collective="allreduce", fp32_matmul=True)
        l32, _ = logits_of(lib32, state)
        check["rounding_floor"] = {"what": "the library arm with every GEMM as an fp32 matmul of the same bf16 operands (another summation order, same "
                                           "rounding points): how far correct implementations drift apart over the layers",
                                   "library_against_it": compare(ref_logits, l32), "ours_against_it": compare(ours_logits, l32)}
        del lib32
        check["status_after"] = eng.check_status()
        del libs

    if not args.no_baseline:
        try:
            library_arm_and_check()
        except Exception as e:          # the headline above stands on its own; a library arm that cannot run is reported, not fatal
            baseline_error = f"{type(e).__name__}: {e}"[:300]

    prof = None
    if args.profile_step and hasattr(eng, "profile_step"):
        eng.profile_step(max_ctx)
        prof = eng.profile_step(max_ctx)

    if rank == 0:
        tok_s = batch * args.steps / (dev_ms * 1e-3)
        e2e_tok_s = batch * args.steps / (e2e_ms * 1e-3)
        hbm = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"] if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 6650.0
        step_bytes = eng.bytes_per_step(ctx + args.warmup + args.steps // 2)
        out = {
            "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (tok_s / baseline["value"]) if baseline else None,
            "dtype": "bf16", "data": "synthetic (random-init weights, N(0,1) KV, uniform context lengths)",
            "config": {"model": cfg.name if args.layers == 36 else f"{cfg.name}-{args.layers}L", "global_batch": batch,
                       "seq_len": f"context uniform {args.ctx_lo}-{args.ctx_hi}, 1 new token per step",
                       "parallelism": f"tp{world}" + (f" ({args.tp_collective})" if world > 1 else ""), "kv_block_tokens": 16, "sampling": "greedy",
                       "attention": f"{args.attn_impl}, {eng.attn.chunk_tokens}-token splits" + ("" if args.attn_chunk or eng.attn.chunk_tokens == 1024 else " (planned from the context lengths)"),
                       "l2": "inputs larger than L2: each step streams %.1f GB of weights and KV per GPU" % (step_bytes / 1e9)},
            "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": sess.h2d_bytes_per_step, "d2h_bytes_per_step": sess.d2h_bytes_per_step},
            "gpu_launches": eng.kernels_per_step * args.steps,
            "clocks": clocks.summary(),
            "roofline": {"hbm_bytes_per_step_per_gpu": step_bytes, "hbm_gbs_achieved": step_bytes / (dev_ms / args.steps) / 1e6,
                         "hbm_frac_of_measured": step_bytes / (dev_ms / args.steps) / 1e6 / hbm},
            "kernel_status": status, "impl": "ours",
        }
        if baseline:
            out["baseline"] = baseline
        if check:
            out["check"] = check
        if baseline_error:
            out["baseline_error"] = baseline_error
        if prof:
            out["eager_step_profile_ms"] = prof
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
