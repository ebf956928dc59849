"""Rank liveness (skygdr_b200/parallel/liveness.py) with real processes on CPU: gloo ranks in lock step, one of which
raises, exits early, crashes or never starts. No GPU is involved and nothing is made to fail on a device."""
import datetime
import json
import os
import socket
import subprocess
import sys

import pytest
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "multi", "liveness_worker.py")


def run_job(world, fail_rank=-1, mode="none", fail_at=3, start=None):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    store = dist.TCPStore("127.0.0.1", port, is_master=True, wait_for_workers=False, timeout=datetime.timedelta(seconds=20))
    procs = {}
    for r in (range(world) if start is None else start):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), STORE_PORT=str(port), FAIL_RANK=str(fail_rank), FAIL_MODE=mode,
                   FAIL_AT=str(fail_at), JOIN_TIMEOUT_S="2" if start is not None else "20")
        procs[r] = subprocess.Popen([sys.executable, WORKER], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, cwd=ROOT)
    res = {}
    for r, p in procs.items():
        try:
            so, se = p.communicate(timeout=90)
        except subprocess.TimeoutExpired:
            p.kill()
            so, se = p.communicate()
        lines = [l for l in so.splitlines() if l.startswith("{")]
        res[r] = (p.returncode, json.loads(lines[-1]) if lines else None, se[-1500:])
    del store
    return res


def test_all_ranks_healthy_run_to_the_end():
    res = run_job(3)
    for r, (rc, out, err) in res.items():
        assert rc == 0 and out["steps"] == 40 and out["seen"] is None, (r, rc, out, err)


@pytest.mark.realtime
@pytest.mark.parametrize("mode,reason", [("raise", "ValueError: rank gave up"), ("exit", "done")])
def test_a_rank_that_leaves_between_steps_is_named_with_its_reason(mode, reason):
    res = run_job(3, fail_rank=1, mode=mode, fail_at=4)
    rc, out, err = res[1]
    assert rc == 0 and out["steps"] == 4, (out, err)
    for r in (0, 2):
        rc, out, err = res[r]
        assert rc == 0 and out is not None, err
        assert out["seen"] is not None and out["seen"]["left"].get("1") == reason, out    # learnt on the host, with the reason
        # a survivor that was already inside the step's collective when the marker appeared may also see the other survivor
        # gone: that one leaves with "PeerLost: ..." as its own reason
        assert all(v.startswith("PeerLost") for k, v in out["seen"]["left"].items() if k != "1"), out
        assert 4 <= out["steps"] <= 5, out                   # at most the step that was already past its guard


@pytest.mark.realtime
def test_a_crashed_rank_is_found_by_its_stale_heartbeat_or_by_the_failed_collective():
    res = run_job(3, fail_rank=2, mode="crash", fail_at=5)
    assert res[2][0] == 17
    for r in (0, 1):
        rc, out, err = res[r]
        assert rc == 0 and out is not None, err
        assert out["seen"] is not None and (out["seen"]["stale"] == [2] or "2" in out["seen"]["left"]), out
        assert out["steps"] <= 6, out


@pytest.mark.realtime
def test_a_rank_that_never_starts_is_reported_missing_instead_of_waited_for():
    res = run_job(3, start=[0, 2])
    for r in (0, 2):
        rc, out, err = res[r]
        assert rc == 0 and out is not None, err
        assert out["seen"]["missing"] == [1] and out["steps"] == 0, out


def test_a_store_that_stops_answering_is_reported_as_its_host_rank_gone():
    """When the process that serves the store dies, every call on the store raises (connection reset, broken pipe). The watch
    turns that into a named rank: the store's host as seen from the others, everybody as seen from the host itself."""
    from skygdr_b200.parallel.liveness import PeerLost, RankWatch

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    store = dist.TCPStore("127.0.0.1", port, is_master=True, wait_for_workers=False, timeout=datetime.timedelta(seconds=5))

    class Gone:
        def check(self, keys):
            raise RuntimeError("Connection reset by peer")

        get = set = check

    w = RankWatch(1, 3, store=store, beat_s=0.05, stale_after_s=0.5, name="gone")
    w.store = Gone()
    h = w.check()
    assert h.stale == [0] and not h.left and not h.missing
    with pytest.raises(PeerLost) as e:
        w.guard()
    assert e.value.health.stale == [0]
    w2 = RankWatch(2, 3, store=store, name="gone2", store_host_rank=2)        # the host itself cannot read its own store any more
    w2.store = Gone()
    assert w2.check().stale == [0, 1]
    w2.leave("x")                                                              # writing the marker fails quietly
    del store
