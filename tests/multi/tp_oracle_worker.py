"""Child process of tests/test_ops_cpu.py (one CPU rank each, gloo, started by torch.distributed.run).

Every rank builds its tensor-parallel shard of the same random Qwen3 weights and runs the plain-PyTorch
tensor-parallel forward; the shards' logits, put side by side, must reproduce the unsharded forward. This pins
the shard layout (which heads, FFN columns, O / down input slices and vocabulary range a rank owns) that the
GPU engines rely on, without a GPU.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skygdr_b200.models import Qwen3Config, Qwen3Weights, reference_forward, reference_forward_tp  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    cfg = Qwen3Config.tiny(layers=2)
    cfg.q_heads, cfg.kv_heads, cfg.ffn = 4 * world, 2 * world, 96 * world
    cfg.vocab = 100 * world + 7                       # the last rank's vocabulary slice is shorter
    full = Qwen3Weights(cfg, "cpu", seed=3, std=0.05)
    shard = Qwen3Weights(cfg, "cpu", seed=3, std=0.05, tp_rank=rank, tp_world=world)
    ids = torch.randint(0, cfg.vocab, (11,), generator=torch.Generator().manual_seed(5))
    want = reference_forward(cfg, full, ids)
    got = reference_forward_tp(cfg, shard, ids)
    assert got.shape == (11, shard.vocab_hi - shard.vocab_lo), got.shape
    ref = want[:, shard.vocab_lo:shard.vocab_hi]
    err = float((got - ref).abs().max() / want.abs().max())
    # the slices cover the vocabulary exactly once
    spans = [None] * world
    dist.all_gather_object(spans, (shard.vocab_lo, shard.vocab_hi))
    covered = spans[0][0] == 0 and spans[-1][1] == cfg.vocab and all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
    # greedy sampling over the shards: the best (value, index) over the ranks is the unsharded argmax unless two logits nearly tie
    val, idx = got.max(-1)
    vals, idxs = [None] * world, [None] * world
    dist.all_gather_object(vals, val)
    dist.all_gather_object(idxs, idx + shard.vocab_lo)
    best = torch.stack(vals).argmax(0)
    picked = torch.stack(idxs).gather(0, best[None])[0]
    top2 = want.topk(2, -1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.05 * want.abs().max()
    agree = bool((picked[clear] == want.argmax(-1)[clear]).all())
    errs = [None] * world
    dist.all_gather_object(errs, err)
    if rank == 0:
        print(json.dumps({"world": world, "rel_err_max": max(errs), "covered": covered, "argmax_agrees": agree, "clear_rows": int(clear.sum())}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
