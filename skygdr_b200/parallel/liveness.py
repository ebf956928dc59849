"""Rank liveness for multi-process engines: who is still there, learnt on the host before the next launch.

The tensor-parallel step's kernels wait (bounded) for stores from every peer, so a step launched after a peer has
gone costs a device time-out and produces nothing. ``RankWatch`` lets the surviving ranks find out on the host,
between steps, with none of their kernels in flight:

* every rank announces itself (``join``): a rank that never shows up is reported instead of waited for forever;
* a background thread stamps a heartbeat into a ``torch.distributed`` store every ``beat_s`` seconds;
* a rank that leaves, whether it is done or an exception unwinds it, writes a ``left`` marker with the reason
  (``with RankWatch(...) as w:`` does this on the way out);
* ``check()`` reads the markers and the heartbeats' age in one pass; ``guard()`` raises ``PeerLost`` naming the ranks.

A rank killed outright writes no marker: its heartbeat going stale (``stale_after_s``) is what the others see.
Heartbeats carry ``time.time()``; all ranks of an engine are processes of one machine (they share NVLink), so they
share the clock. The store is any c10d store: the process group's own (default) or a ``TCPStore`` of the caller.

The reference has no liveness or membership of any kind: its programs exit on the first error
(src/cpu_client.cc:38-42) and its server just takes the next client (src/gpu_server.cu:523-530).
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch.distributed as dist


class PeerLost(RuntimeError):
    def __init__(self, health: "Health"):
        super().__init__(f"peers lost: left={health.left} stale={health.stale} missing={health.missing}")
        self.health = health


@dataclass
class Health:
    left: Dict[int, str] = field(default_factory=dict)     # rank -> reason it gave
    stale: List[int] = field(default_factory=list)         # heartbeat older than stale_after_s
    missing: List[int] = field(default_factory=list)       # never announced itself

    @property
    def ok(self) -> bool:
        return not (self.left or self.stale or self.missing)


class RankWatch:
    def __init__(self, rank: int, world: int, store=None, beat_s: float = 0.1, stale_after_s: float = 1.5, name: str = "engine",
                 store_host_rank: int = 0):
        """store_host_rank: the rank whose process serves the store (rank 0 for a store created by ``init_process_group`` from
        a tcp:// address; under torchrun the launcher serves it and it outlives every rank). When the store stops answering,
        that rank is what has gone, and ``check`` reports it as stale instead of raising the store's own error."""
        self.store_host_rank = store_host_rank
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = dist.PrefixStore(f"skygdr_live/{name}", store)
        self.rank, self.world, self.beat_s, self.stale_after_s = rank, world, beat_s, stale_after_s
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._joined = False

    # ---- this rank's side ----
    def _beat(self) -> None:
        self.store.set(f"hb/{self.rank}", repr(time.time()))

    def _run(self) -> None:
        while not self._stop.wait(self.beat_s):
            try:
                self._beat()
            except Exception:           # the store went away with rank 0: the others see this rank go stale, which is the truth
                return

    def join(self, timeout_s: float = 30.0) -> Health:
        """Announces this rank, starts its heartbeat and waits until every rank has announced itself or ``timeout_s`` has
        passed. Returns who is missing (and who has already left again); raises nothing."""
        self._beat()
        self.store.set(f"joined/{self.rank}", "1")
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="skygdr-rankwatch", daemon=True)
            self._thread.start()
        self._joined = True
        deadline = time.monotonic() + timeout_s
        while True:
            missing = [r for r in range(self.world) if not self.store.check([f"joined/{r}"])]
            if not missing or time.monotonic() > deadline:
                h = self.check()
                h.missing = missing
                h.stale = [r for r in h.stale if r not in missing]
                return h
            time.sleep(min(0.05, self.beat_s))

    def leave(self, reason: str = "done") -> None:
        """Marks this rank as gone. Call it between steps, with none of this rank's kernels or collectives in flight."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            self._thread = None
        try:
            self.store.set(f"left/{self.rank}", reason[:200] or "done")
        except Exception:
            pass

    # ---- the others' side ----
    def check(self) -> Health:
        """One pass over the peers' markers and heartbeats; does not block. A store that no longer answers (its host process
        is gone) is not an error of this rank: the host rank is reported as stale, so that ``guard`` raises ``PeerLost``."""
        h, now = Health(), time.time()
        try:
            for r in range(self.world):
                if r == self.rank:
                    continue
                if self.store.check([f"left/{r}"]):
                    h.left[r] = self.store.get(f"left/{r}").decode()
                elif not self.store.check([f"hb/{r}"]):
                    h.missing.append(r)
                elif now - float(self.store.get(f"hb/{r}").decode()) > self.stale_after_s:
                    h.stale.append(r)
        except Exception:               # connection reset / broken pipe / store timeout: the store's host has gone
            lost = self.store_host_rank if self.store_host_rank != self.rank else None
            if lost is not None and lost not in h.stale and lost not in h.left:
                h.stale.append(lost)
            elif lost is None:          # this rank hosts the store and cannot read it: nothing about the peers can be known
                h.stale = [r for r in range(self.world) if r != self.rank and r not in h.left]
        return h

    def guard(self) -> None:
        """Call before launching a step: raises ``PeerLost`` if any peer has left, gone silent or never joined."""
        h = self.check()
        if not h.ok:
            raise PeerLost(h)

    def __enter__(self) -> "RankWatch":
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        self.leave("done" if exc_type is None else f"{exc_type.__name__}: {exc}")
        return False
