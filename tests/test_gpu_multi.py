"""Multi-GPU checks, run as child processes (one per GPU). Skipped below 2 GPUs."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world, script, timeout=240, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "multi", script)]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


def _why(r) -> str:
    """What a failed child run said: its own TP_WORKER_FAIL lines first (the launcher's summary hides them), then the tails."""
    own = [ln for ln in r.stdout.splitlines() if "TP_WORKER_FAIL" in ln]
    return "\n".join(own[:8]) + "\n" + r.stdout[-2000:] + r.stderr[-2000:]


def _gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("collective", ["oneshot", "rs_ag"])
def test_tensor_parallel_decode_and_peer_kv_transfer(world, collective):
    """The tensor-parallel decoder against the single-GPU decoder, step by step (eager and as a replayed graph), in both
    collective forms and at every world size the box has GPUs for; plus a paged KV transfer between two ranks."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    r = _run(world, "tp_worker.py", SKYGDR_TP_COLLECTIVE=collective)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, _why(r)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_decode_at_the_model_widths(world):
    """Two layers of the Qwen3-8B widths (hidden 4096, 32 / 8 heads, FFN 12288), 16 sequences per rank: the tile shapes,
    split factors and arrival counts of the benchmark, checked against the single-GPU decoder."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    r = _run(world, "tp_worker.py", timeout=400, SKYGDR_TP_SHAPE="real")
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, _why(r)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_a_rank_leaving_between_steps_is_learnt_on_the_host_before_the_next_launch():
    """Rank world-1 leaves a tensor-parallel job between steps (nothing in flight); the others must get PeerLost from the
    liveness store instead of launching a step that would wait for it, and keep a usable context."""
    r = _run(2, "tp_leave_worker.py")
    assert "TP_LEAVE_LEFT" in r.stdout and "TP_LEAVE_DETECTED rank=0" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 3, reason="needs 3 GPUs (source + 2 destinations)")
def test_multicast_fanout_lands_in_every_destination():
    """GPU0's pages go out once through the NVLink multicast address and must equal, in both destinations' pools, what
    the unicast fan-out writes (a PyTorch permute of the source pages). One process drives the three GPUs."""
    from skygdr_b200 import ops
    from skygdr_b200._ext import load

    C = load()
    ok, why = C.multicast_supported(0)
    if not ok:
        pytest.skip(f"no NVLink multicast here: {why}")
    geom = ops.KVGeometry(layers=3, kv_heads=8)
    nb = 40
    src = ops.PagedKVPool(geom, nb, "nhd", device="cuda:0")
    src.data.normal_()
    g = torch.Generator().manual_seed(5)
    sp = torch.randperm(nb, generator=g).int().cuda(0)
    dp = torch.randperm(nb, generator=g).int().cuda(0)
    with ops.MulticastPools(geom, nb, [0, 1, 2]) as mc:
        for pool in mc.pools:
            pool.data.fill_(-1.0)
        for d in range(3):
            torch.cuda.synchronize(d)
        flow = ops.KvTransferFlow("cuda:0", method="simt")
        none = [ops.RemotePool(0, mc.pools[0].strides, geom.kv_heads) for _ in range(2)]
        with torch.cuda.device(0):
            flow.transfer(src, none, sp[:32], dp[:32], replicate=True, multicast_ptr=mc.multicast_ptr)
            st = flow.result()
        assert st["status"] == 0 and st["bytes_done"] == ops.link_bytes(geom, 32)        # egress counts the payload once
        want = ops.reference_transfer(src, sp[:32])
        for pool in mc.pools:                                                              # the source's own copy receives it too
            dev = pool.data.device
            assert torch.equal(pool.data[dp[:32].long().to(dev)], want.to(dev))
            untouched = dp[32:].long().to(dev)
            assert bool((pool.data[untouched] == -1.0).all())


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 3, reason="needs 3 GPUs (source + 2 destinations)")
@pytest.mark.parametrize("prefer_multicast", [True, False])
def test_fanout_target_sends_the_same_way_with_and_without_multicast(prefer_multicast):
    """FanoutTarget picks the NVLink multicast address where it exists and unicast peer stores otherwise; the destinations
    end up with the same pages either way."""
    from skygdr_b200 import ops

    geom = ops.KVGeometry(layers=2, kv_heads=8)
    src = ops.PagedKVPool(geom, 24, "nhd", device="cuda:0")
    src.data.normal_()
    sb = torch.arange(16, device="cuda:0").int()
    db = (torch.arange(16, device="cuda:0") + 4).int()
    with ops.FanoutTarget(geom, 24, 0, [1, 2], prefer_multicast=prefer_multicast) as tgt:
        assert tgt.mode in ("multimem", "unicast") and (prefer_multicast or tgt.mode == "unicast")
        flow = ops.KvTransferFlow("cuda:0", method="simt")
        with torch.cuda.device(0):
            tgt.send(flow, src, sb, db)
            st = flow.result()
        assert st["status"] == 0
        want = ops.reference_transfer(src, sb)
        for pool in tgt.pools:
            dev = pool.data.device
            assert torch.equal(pool.data[db.long().to(dev)], want.to(dev))
