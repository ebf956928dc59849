"""KV hand-off through a collective library's send / recv: the comparison arm of benchmarks/config2_kv_transfer.py for
stacks that move KV with NCCL instead of a transfer kernel.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29541 \
        benchmarks/config2_library_sendrecv.py [--requests 12] [--out results/config2_library.json]

Rank 0 sends, rank 1 receives; the same workload as config 2 (Qwen3-8B-shaped paged KV, 16-token blocks, randomly
permuted block tables, sequence lengths uniform 1k-64k, same seed). Arms:
  send_recv_paged        gather + layout change into staging, send, scatter into the destination's blocks (what a
                         paged cache needs; functionally what the transfer kernel does in one launch)
  send_recv_contiguous   one contiguous region per request, no block table, no layout change (the library's best case)
On GPUs every time is a device time (CUDA events on each rank around the request, maximum over the two ranks);
``--device cpu`` runs the same code over gloo with wall-clock times, which is only good for checking the logic.
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from skygdr_b200.ops.kv_cache import KVGeometry, PagedKVPool  # noqa: E402
from skygdr_b200.parallel.library_handoff import LibraryKvHandoff  # noqa: E402

NVLINK_NOMINAL, NVLINK_MEASURED = 900.0, 770.0


def filled_pool(geom, n, layout, dev, seed):
    """The same values on every rank: generated on the CPU in slices from one seed."""
    pool = PagedKVPool(geom, n, layout, device=dev)
    g = torch.Generator().manual_seed(seed)
    for i in range(0, n, 64):
        m = min(64, n - i)
        pool.data[i:i + m].copy_(torch.randn((m,) + tuple(pool.data.shape[1:]), generator=g).to(pool.data.dtype))
    return pool


class Timer:
    def __init__(self, dev):
        self.cuda = dev.type == "cuda"
        if self.cuda:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        if self.cuda:
            self.e0.record()
        else:
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            self.e1.record()
            self.e1.synchronize()
            self.seconds = self.e0.elapsed_time(self.e1) * 1e-3
        else:
            self.seconds = time.perf_counter() - self.t0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=12)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--min-tokens", type=int, default=1024)
    ap.add_argument("--max-tokens", type=int, default=65536)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--blocks-per-message", type=int, default=64)
    ap.add_argument("--device", default="cuda", choices=("cuda", "cpu"))
    ap.add_argument("--out", default="results/config2_library.json")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    assert world == 2, "one sending and one receiving rank: start with --nproc-per-node 2"
    if a.device == "cuda":
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")

    geom = KVGeometry(layers=a.layers)
    g = torch.Generator().manual_seed(a.seed)
    seq = torch.randint(a.min_tokens, a.max_tokens + 1, (a.requests,), generator=g).tolist()
    blocks = [geom.blocks_for(t) for t in seq]
    max_blocks = max(blocks)
    g2 = torch.Generator().manual_seed(a.seed)
    sp = torch.randperm(max_blocks, generator=g2).to(dev)
    dp = torch.randperm(max_blocks, generator=g2).to(dev)

    # ---- correctness on a small pool that both ranks can build: the receiver knows what it must end up holding ----
    nv = min(96, max_blocks)
    small_src = filled_pool(geom, nv, "nhd", dev, a.seed + 1)
    vs, vd = torch.randperm(nv, generator=g2).to(dev), torch.randperm(nv, generator=g2).to(dev)
    exact = True
    if rank == 0:
        LibraryKvHandoff(small_src, min(a.blocks_per_message, 40)).send_paged(vs, 1)
    else:
        small_dst = PagedKVPool(geom, nv, "hnd", device=dev)
        LibraryKvHandoff(small_dst, min(a.blocks_per_message, 40)).recv_paged(vd, 0)
        want = small_src.data[vs].permute(0, 1, 2, 4, 3, 5)
        exact = bool(torch.equal(small_dst.data[vd], want))
    del small_src

    # ---- timing ----
    layout = "nhd" if rank == 0 else "hnd"
    pool = PagedKVPool(geom, max_blocks, layout, device=dev)
    if rank == 0:
        for i in range(0, max_blocks, 256):
            pool.data[i:i + 256].normal_()
    hand = LibraryKvHandoff(pool, a.blocks_per_message)
    res = {}
    for arm in ("send_recv_paged", "send_recv_contiguous"):
        tot_b, tot_s = 0, 0.0
        for i, nb in enumerate([blocks[0]] + blocks):           # the first one warms up (communicator set-up, allocator)
            dist.barrier()
            with Timer(dev) as t:
                if arm == "send_recv_paged":
                    n = hand.send_paged(sp[:nb], 1) if rank == 0 else hand.recv_paged(dp[:nb], 0)
                else:
                    n = hand.send_contiguous(nb, 1) if rank == 0 else hand.recv_contiguous(nb, 0)
            sec = torch.tensor([t.seconds], dtype=torch.float64, device=dev)
            dist.all_reduce(sec, op=dist.ReduceOp.MAX)           # a request is done when the slower side is done
            if i >= 1:
                tot_b += n
                tot_s += float(sec.item())
        gbs = tot_b / tot_s / 1e9
        res[arm] = {"gb": tot_b / 1e9, "gbs": gbs, "frac_of_900": gbs / NVLINK_NOMINAL, "frac_of_measured_770": gbs / NVLINK_MEASURED}
    flag = torch.tensor([1 if exact else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    res["send_recv_paged"]["exact"] = bool(flag.item())
    if rank == 0:
        out = {"config": {"geometry": f"{a.layers} layers x 8 kv heads x 128, bf16, 16-token blocks", "seq_lens": seq,
                          "blocks_per_message": a.blocks_per_message, "backend": dist.get_backend(), "timing": "cuda events, max over ranks" if a.device == "cuda" else "wall clock (logic check only)"},
               "arms": res}
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        json.dump(out, open(a.out, "w"), indent=1)
        print(json.dumps(res, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
