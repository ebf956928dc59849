"""Paged KV pools.

A pool holds ``num_blocks`` blocks of 16 tokens for every layer, K and V:

* ``nhd`` (token-major, prefill side):  [block][layer][2][16 tok][H][128]
* ``hnd`` (head-major, decode side):    [block][layer][2][H][16 tok][128]

so one block is one contiguous range on both sides, and in ``hnd`` a page of
one head is one contiguous 4 KiB range, which is what the attention kernel's
bulk copies fetch. The reference keeps KV as one flat array per run with no
block table (llm_problem_analysis/decode_vllm_kvcache_hbm_stress.cu:154-168).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

BLOCK_TOKENS = 16


@dataclass
class KVGeometry:
    layers: int = 36
    kv_heads: int = 8
    head_dim: int = 128
    block_tokens: int = BLOCK_TOKENS

    @property
    def page_elems(self) -> int:
        return self.block_tokens * self.kv_heads * self.head_dim

    @property
    def block_elems(self) -> int:
        return self.layers * 2 * self.page_elems

    def bytes_per_token(self, elem_bytes: int = 2) -> int:
        return self.layers * 2 * self.kv_heads * self.head_dim * elem_bytes

    def blocks_for(self, tokens: int) -> int:
        return (tokens + self.block_tokens - 1) // self.block_tokens


class PagedKVPool:
    def __init__(self, geom: KVGeometry, num_blocks: int, layout: str = "hnd", device="cuda", dtype=torch.bfloat16,
                 data: Optional[torch.Tensor] = None):
        assert layout in ("nhd", "hnd")
        self.geom, self.num_blocks, self.layout = geom, num_blocks, layout
        g = geom
        shape = ((num_blocks, g.layers, 2, g.block_tokens, g.kv_heads, g.head_dim) if layout == "nhd"
                 else (num_blocks, g.layers, 2, g.kv_heads, g.block_tokens, g.head_dim))
        if data is None:
            data = torch.zeros(shape, dtype=dtype, device=device)
        else:
            data = data.view(shape)
        self.data = data

    # strides in elements: (block, layer, kv)
    @property
    def strides(self) -> Tuple[int, int, int]:
        s = self.data.stride()
        return (s[0], s[1], s[2])

    @property
    def head_stride(self) -> int:
        assert self.layout == "hnd"
        return self.data.stride(3)

    def layer_base(self, layer: int) -> torch.Tensor:
        """1-element-offset view whose data_ptr is the first page of ``layer`` in block 0."""
        return self.data[0, layer]

    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()

    def gather_reference(self, blocks: torch.Tensor) -> torch.Tensor:
        """[n][layer][2][tok][head][dim] in token-major order whatever the pool's layout (for tests)."""
        x = self.data[blocks.long()]
        return x if self.layout == "nhd" else x.permute(0, 1, 2, 4, 3, 5).contiguous()


class BlockAllocator:
    """Free list over a pool's blocks and the block tables that the kernels read.

    ``table`` is the int32 [max_seqs][max_blocks] tensor handed to the attention, append and transfer kernels (kept on the
    host side here; copy it to the device when it changes). A sequence slot owns the blocks listed in its row; ``ensure``
    grows a row to cover a context length and ``release`` returns a slot's blocks. Block 0 can be kept out of circulation so
    that unused table entries (zeros) never alias live data. The reference has no paging at all
    (llm_problem_analysis/decode_vllm_kvcache_hbm_stress.cu:154-168 indexes one flat array)."""

    def __init__(self, num_blocks: int, max_seqs: int, max_ctx: int, block_tokens: int = BLOCK_TOKENS, reserve_block0: bool = True):
        self.block_tokens = block_tokens
        self.max_blocks = (max_ctx + block_tokens - 1) // block_tokens
        first = 1 if reserve_block0 else 0
        self._free = list(range(num_blocks - 1, first - 1, -1))       # pop() hands out low ids first
        self.capacity = len(self._free)
        self.table = torch.zeros((max_seqs, self.max_blocks), dtype=torch.int32)
        self.n_blocks = [0] * max_seqs

    @property
    def free_blocks(self) -> int:
        return len(self._free)

    def blocks_for(self, tokens: int) -> int:
        return (tokens + self.block_tokens - 1) // self.block_tokens

    def can_fit(self, slot: int, tokens: int) -> bool:
        need = self.blocks_for(tokens)
        return need <= self.max_blocks and need - self.n_blocks[slot] <= len(self._free)

    def ensure(self, slot: int, tokens: int) -> int:
        """Makes slot's row cover ``tokens`` tokens; returns how many blocks were added. Raises MemoryError, leaving the row as
        it was, when the pool (or the row) cannot hold them."""
        need = self.blocks_for(tokens)
        have = self.n_blocks[slot]
        if need <= have:
            return 0
        if need > self.max_blocks:
            raise MemoryError(f"{tokens} tokens need {need} blocks, a table row holds {self.max_blocks}")
        if need - have > len(self._free):
            raise MemoryError(f"{need - have} blocks wanted, {len(self._free)} free")
        for i in range(have, need):
            self.table[slot, i] = self._free.pop()
        self.n_blocks[slot] = need
        return need - have

    def blocks_of(self, slot: int) -> torch.Tensor:
        return self.table[slot, :self.n_blocks[slot]].clone()

    def release(self, slot: int) -> int:
        n = self.n_blocks[slot]
        self._free.extend(reversed(self.table[slot, :n].tolist()))
        self.table[slot, :n] = 0
        self.n_blocks[slot] = 0
        return n
