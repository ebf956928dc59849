"""Child process of tests/test_parallel_liveness.py: one CPU rank of a small lock-step job (gloo), started directly
by the test (no launcher that would tear the others down when one exits). The test process hosts the store.

Environment: RANK, WORLD_SIZE, STORE_PORT, FAIL_RANK, FAIL_MODE (none | raise | exit | crash | never_join), FAIL_AT.
Every failure is made on the host, between steps: an exception, a clean exit, an abrupt exit, a rank that is never
started. Survivors must notice before their next step, or have that step's collective end with an error, report
what they saw as one JSON line and exit 0.
"""
import datetime
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skygdr_b200.parallel.liveness import PeerLost, RankWatch  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    fail_rank, mode, fail_at = int(os.environ.get("FAIL_RANK", "-1")), os.environ.get("FAIL_MODE", "none"), int(os.environ.get("FAIL_AT", "3"))
    store = dist.TCPStore("127.0.0.1", int(os.environ["STORE_PORT"]), is_master=False, timeout=datetime.timedelta(seconds=20))
    out = {"rank": rank, "steps": 0, "seen": None, "collective_error": False}
    watch = RankWatch(rank, world, store=store, beat_s=0.05, stale_after_s=0.6, name="job")
    h = watch.join(timeout_s=float(os.environ.get("JOIN_TIMEOUT_S", "3")))
    if not h.ok:                                             # somebody never came: do not even build the process group
        out["seen"] = {"missing": h.missing, "left": h.left, "stale": h.stale}
        watch.leave("peer missing at start")
        print(json.dumps(out), flush=True)
        return 0
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    x = torch.ones(4)
    try:
        with watch:
            for step in range(40):
                if rank == fail_rank and step == fail_at:
                    if mode == "raise":
                        raise ValueError("rank gave up")     # the context manager writes the marker on the way out
                    if mode == "exit":
                        break                                # a clean early exit: marker "done"
                    if mode == "crash":
                        sys.stdout.flush()
                        os._exit(17)                         # no marker, no goodbye: the heartbeat just stops
                watch.guard()
                try:
                    dist.all_reduce(x)                       # "the step"
                except RuntimeError:
                    # the peer vanished after the guard: the short process-group timeout (or the closed socket) ends the
                    # collective with an error; the next guard names the rank once its heartbeat has gone stale
                    out["collective_error"] = True
                    deadline = time.monotonic() + 3.0
                    while time.monotonic() < deadline:
                        watch.guard()
                        time.sleep(0.05)
                    raise
                out["steps"] = step + 1
                time.sleep(0.02)
    except PeerLost as e:
        out["seen"] = {"missing": e.health.missing, "left": e.health.left, "stale": e.health.stale}
    except ValueError as e:
        out["raised"] = str(e)
    print(json.dumps(out), flush=True)
    os._exit(0)        # the process group may hold sockets to a dead peer: leave without its teardown


if __name__ == "__main__":
    sys.exit(main())
