"""Comparison arm for the KV-transfer kernel: the same hand-off through a collective library's send / recv.

A serving stack without a transfer kernel of its own moves a paged KV cache between two ranks in three steps:
gather the request's blocks into a contiguous staging buffer (and change the layout there), send it with the
library (``torch.distributed`` send / recv: NCCL over NVLink on GPUs), scatter it into the destination's blocks.
``LibraryKvHandoff`` does exactly that, chunked so that the staging buffers stay small, and also offers the best case
for the library, one contiguous region with no block table and no layout change, which is what the reference's
``cudaMemcpyPeerAsync`` loop moves (llm_problem_analysis/kv_nvlink_transfer.cu:113-137).

This is the baseline mechanism, not the product path: ``ops.KvTransferFlow`` does gather, layout change and the
peer stores in one kernel with no staging and no second pass over HBM on either side.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops.kv_cache import PagedKVPool


class LibraryKvHandoff:
    """One direction of a hand-off between two ranks of ``group``. Both sides construct it with the same
    ``blocks_per_message``; the sender calls ``send_*``, the receiver the matching ``recv_*``."""

    def __init__(self, pool: PagedKVPool, blocks_per_message: int = 64, group=None):
        assert blocks_per_message >= 1
        self.pool, self.bpm, self.group = pool, blocks_per_message, group
        g = pool.geom
        # head-major staging, two buffers so that the gather (or scatter) of one message overlaps the wire time of the other
        shape = (blocks_per_message, g.layers, 2, g.kv_heads, g.block_tokens, g.head_dim)
        self.stage = [torch.empty(shape, dtype=pool.data.dtype, device=pool.data.device) for _ in range(2)]

    # ---- paged: what the transfer kernel does, in library calls ----
    def send_paged(self, blocks: torch.Tensor, dst: int) -> int:
        """Gathers ``blocks`` of a token-major (or head-major) pool into head-major staging and sends them. Returns bytes sent."""
        idx = blocks.long()
        pending: list = [None, None]
        sent = 0
        for i, lo in enumerate(range(0, idx.numel(), self.bpm)):
            part = idx[lo:lo + self.bpm]
            buf = self.stage[i & 1][: part.numel()]
            if pending[i & 1] is not None:
                pending[i & 1].wait()                       # the buffer's previous message has left
            x = self.pool.data[part]
            buf.copy_(x.permute(0, 1, 2, 4, 3, 5) if self.pool.layout == "nhd" else x)
            pending[i & 1] = dist.isend(buf, dst, group=self.group)
            sent += buf.numel() * buf.element_size()
        for w in pending:
            if w is not None:
                w.wait()
        return sent

    def recv_paged(self, blocks: torch.Tensor, src: int) -> int:
        """Receives what ``send_paged`` sends and scatters it into ``blocks`` of a head-major pool. Returns bytes received."""
        assert self.pool.layout == "hnd", "the decode side keeps head-major pages"
        idx = blocks.long()
        parts = [idx[lo:lo + self.bpm] for lo in range(0, idx.numel(), self.bpm)]
        got = 0
        work: Optional[object] = None
        if parts:
            work = dist.irecv(self.stage[0][: parts[0].numel()], src, group=self.group)
        for i, part in enumerate(parts):
            work.wait()
            nxt = None
            if i + 1 < len(parts):                          # post the next receive before scattering this one
                nxt = dist.irecv(self.stage[(i + 1) & 1][: parts[i + 1].numel()], src, group=self.group)
            buf = self.stage[i & 1][: part.numel()]
            self.pool.data.index_copy_(0, part, buf)
            got += buf.numel() * buf.element_size()
            work = nxt
        return got

    # ---- contiguous: the library's best case (no block table, no layout change) ----
    def send_contiguous(self, n_blocks: int, dst: int) -> int:
        x = self.pool.data[:n_blocks]
        dist.send(x, dst, group=self.group)
        return x.numel() * x.element_size()

    def recv_contiguous(self, n_blocks: int, src: int) -> int:
        x = self.pool.data[:n_blocks]
        dist.recv(x, src, group=self.group)
        return x.numel() * x.element_size()
