"""Child process of tests/test_gpu_multi.py (one per GPU): a rank leaves a tensor-parallel decode job between steps.

The leaving rank synchronises its device first (none of its kernels in flight), writes its marker and exits. The
other ranks learn of it on the host, through the liveness store, before their next launch: the step is never
launched, no kernel waits for the missing peer, and their context stays usable. Plain peer stores only; NVLS off.
"""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skygdr_b200 import ops  # noqa: E402
from skygdr_b200.models import Qwen3Config, Qwen3Weights  # noqa: E402
from skygdr_b200.parallel.liveness import PeerLost, RankWatch  # noqa: E402
from skygdr_b200.parallel.tp import TPDecoder  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = Qwen3Config.tiny(layers=2)
    cfg.kv_heads, cfg.q_heads, cfg.ffn, cfg.vocab = 2 * world, 8 * world, 256 * world, 256 * world
    w = Qwen3Weights(cfg, dev, seed=3, std=0.05, tp_rank=rank, tp_world=world)
    B, max_ctx = 2 * world, 128
    pool = ops.PagedKVPool(ops.KVGeometry(cfg.layers, cfg.kv_heads // world, cfg.head_dim), B * 8 + 1, "hnd", device=dev)
    tp = TPDecoder(cfg, w, pool, B, max_ctx, rank, world, attn_chunk=128)
    table = (torch.arange(B * 8, dtype=torch.int32).view(B, 8) + 1).to(dev)
    tp.set_batch(torch.arange(B, dtype=torch.int32, device=dev), torch.full((B,), 20, dtype=torch.int32, device=dev), table)
    watch = RankWatch(rank, world, beat_s=0.05, stale_after_s=1.0, name="tp_leave")
    assert watch.join(timeout_s=30).ok
    tp.attach_watch(watch)
    for _ in range(3):
        tp.step(max_ctx=max_ctx)
    assert tp.check_status() == "OK"                         # synchronises: nothing of this rank is in flight
    dist.barrier()
    torch.cuda.synchronize(dev)
    if rank == world - 1:
        watch.leave("done")
        print("TP_LEAVE_LEFT", flush=True)
        os._exit(0)
    deadline = time.monotonic() + 10
    while watch.check().ok and time.monotonic() < deadline:  # host only: wait until the marker is in the store
        time.sleep(0.02)
    try:
        tp.step(max_ctx=max_ctx)                             # must raise before anything is launched
        raise AssertionError("a step was launched although a peer had left")
    except PeerLost as e:
        assert e.health.left.get(world - 1) == "done", e.health
    assert tp.check_status() == "OK"                         # no kernel waited for the missing rank; the context is fine
    y = torch.ones(8, device=dev).sum().item()
    assert y == 8.0
    watch.leave("peer lost")
    print(f"TP_LEAVE_DETECTED rank={rank}", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
