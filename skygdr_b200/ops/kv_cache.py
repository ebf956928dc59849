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
