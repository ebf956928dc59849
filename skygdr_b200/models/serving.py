"""Continuous batching over a decode engine: requests come and go while the batch keeps stepping.

The engine (``Qwen3Decoder`` or anything with the same four calls) has a fixed number of batch slots and reads, per
slot, the token to feed, its position and a block-table row. ``ContinuousBatcher`` owns the slots and the pool's
blocks (``ops.BlockAllocator``):

* ``submit`` queues a request; a request is admitted when a slot is free and the allocator can hold its prompt plus
  everything it may generate (blocks are reserved up front, so a running request is never evicted);
* admission prefills the prompt into the request's blocks and takes the first token from the prefill logits;
* every ``step`` feeds each running sequence its last token, runs ONE engine step over all slots and appends the
  sampled tokens; idle slots run along on block 0, which the allocator keeps out of circulation, so the engine's
  batch shape (and a captured CUDA graph) never changes;
* a sequence ends at ``max_new_tokens`` or at its ``eos_id``; its slot and blocks are free for the next admission.

The reference has no serving loop (its case study drives vLLM, README.md:56-75); this is the host-side scheduler that
the prefill / decode engines of this package need to serve more than one fixed batch.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple

import torch

from ..ops.kv_cache import BlockAllocator


@dataclass
class Request:
    req_id: int
    prompt: torch.Tensor                     # int token ids, 1-D, at least one
    max_new_tokens: int
    eos_id: Optional[int] = None
    output: List[int] = field(default_factory=list)
    finished: bool = False


class ContinuousBatcher:
    def __init__(self, engine, allocator: BlockAllocator, use_graph: bool = True):
        """use_graph: run the decode step as a replay of the engine's captured CUDA graph when the engine can capture one (the
        step is launch-bound otherwise); the batch shape never changes, so one capture serves every step."""
        self.eng, self.alloc = engine, allocator
        self._graph = bool(use_graph and hasattr(engine, "capture") and hasattr(engine, "replay"))
        self.slots: List[Optional[Request]] = [None] * engine.max_batch
        assert allocator.table.shape[0] >= engine.max_batch, "one table row per engine slot"
        self.waiting: Deque[Request] = deque()
        self.h_ids = torch.zeros(engine.max_batch, dtype=torch.int32)
        self.h_pos = torch.zeros(engine.max_batch, dtype=torch.int32)
        self.steps = 0

    # ---- queue ----
    def submit(self, req: Request) -> None:
        assert req.prompt.numel() >= 1 and req.max_new_tokens >= 1
        total = int(req.prompt.numel()) + req.max_new_tokens
        if self.alloc.blocks_for(total) > min(self.alloc.max_blocks, self.alloc.capacity):
            raise MemoryError(f"request {req.req_id}: {total} tokens can never fit this pool")
        self.waiting.append(req)

    @property
    def running(self) -> int:
        return sum(r is not None for r in self.slots)

    def idle(self) -> bool:
        return not self.waiting and self.running == 0

    # ---- admission: first come first served; the head of the queue is never overtaken ----
    def _admit(self) -> List[Tuple[int, int]]:
        out = []
        while self.waiting:
            req = self.waiting[0]
            free = [i for i, r in enumerate(self.slots) if r is None]
            total = int(req.prompt.numel()) + req.max_new_tokens
            if not free or not self.alloc.can_fit(free[0], total):
                break
            self.waiting.popleft()
            slot = free[0]
            self.alloc.ensure(slot, total)
            n = int(req.prompt.numel())
            dev = self.eng.device
            row = self.alloc.table[slot:slot + 1].to(dev)
            logits = self.eng.prefill(req.prompt.to(dev), [n], row)
            tok = int(logits.float().argmax(-1)[0])
            self.slots[slot] = req
            self.h_pos[slot] = n                     # the first generated token sits at position n
            out += self._accept(slot, tok)
        return out

    def _accept(self, slot: int, tok: int) -> List[Tuple[int, int]]:
        req = self.slots[slot]
        req.output.append(tok)
        self.h_ids[slot] = tok
        if len(req.output) >= req.max_new_tokens or (req.eos_id is not None and tok == req.eos_id):
            req.finished = True
            self.slots[slot] = None
            self.alloc.release(slot)
            self.h_ids[slot] = 0
            self.h_pos[slot] = 0
        return [(req.req_id, tok)]

    # ---- one scheduling round: admit what fits, then one engine step over all slots ----
    def step(self) -> List[Tuple[int, int]]:
        out = self._admit()
        if self.running == 0:
            return out
        dev = self.eng.device
        self.eng.set_batch(self.h_ids.to(dev), self.h_pos.to(dev), self.alloc.table[:self.eng.max_batch].to(dev))
        if self._graph:
            if getattr(self.eng, "graph", None) is None or getattr(self.eng, "graph_batch", None) != self.eng.max_batch:
                self.eng.capture(self.eng.max_batch, self.eng.max_ctx)
            nxt = self.eng.replay().cpu()
        else:
            nxt = self.eng.step().cpu()
        self.steps += 1
        for slot, req in enumerate(self.slots):
            if req is None:
                continue
            self.h_pos[slot] += 1
            out += self._accept(slot, int(nxt[slot]))
        return out

    def run_until_idle(self, max_steps: int = 1 << 30) -> Dict[int, List[int]]:
        done: Dict[int, List[int]] = {}
        for _ in range(max_steps):
            if self.idle():
                break
            for rid, tok in self.step():
                done.setdefault(rid, []).append(tok)
        return done
