"""Paged GQA decode attention (skygdr_b200/csrc/kernels/paged_attn.cu)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .._ext import load
from .flow import new_status
from .kv_cache import PagedKVPool


def simulate_decode_launch(ctx_lens, kv_heads: int, chunk_tokens: int, slots: int = 296, hbm_bytes_per_us: float = 6.0e6,
                           cta_bytes_per_us: float = 80e3, setup_us: float = 1.5, finish_us: float = 1.0) -> float:
    """Microseconds one launch of the tcgen05 decode kernel takes, by a fluid model: one CTA per (sequence, KV head, chunk) in the
    kernel's dispatch order (chunks fastest, then heads, then sequences), `slots` of them resident (two per SM), each setting
    up, then streaming its tiles of 128 tokens (64 KB of K and V) at an equal share of the memory bandwidth but no faster than
    one CTA's ring allows, then finishing. The absolute figure is about 35 us short of a measured launch; what it is used for is
    the order of the candidates, which it got right where it was checked on B200 (contexts 8k-16k: 2048 < 1536 < 1024 < 768 < 512
    tokens per chunk, measured 167.7 / 170.6 / 171.5 / 173.3 / 183.6 us; the benchmark's contexts 2k-16k: 1536 ahead of 1024 and
    2048 by 2.4 % of the decode step)."""
    items = []
    for c in ctx_lens:
        c = int(c)
        n = (c + chunk_tokens - 1) // chunk_tokens
        sizes = [((min(c, (s + 1) * chunk_tokens) - s * chunk_tokens + 127) // 128) * 65536.0 for s in range(n)]
        for _ in range(kv_heads):
            items.extend(sizes)
    t, nxt = 0.0, 0
    active = []                                  # [bytes left, set-up left, finish left]
    while nxt < len(items) or active:
        while len(active) < slots and nxt < len(items):
            active.append([items[nxt], setup_us, finish_us])
            nxt += 1
        streaming = sum(1 for a in active if a[1] <= 0 and a[0] > 0)
        rate = min(cta_bytes_per_us, hbm_bytes_per_us / max(1, streaming))
        dt = min(a[1] if a[1] > 0 else (a[0] / rate if a[0] > 0 else a[2]) for a in active)
        for a in active:
            if a[1] > 0:
                a[1] = a[1] - dt if a[1] - dt > 1e-9 else 0.0
            elif a[0] > 0:
                a[0] = a[0] - dt * rate if a[0] - dt * rate > 1e-6 else 0.0
            else:
                a[2] -= dt
        active = [a for a in active if a[1] > 0 or a[0] > 0 or a[2] > 1e-9]
        t += dt
    return t


def plan_chunk_tokens(ctx_lens, kv_heads: int, sms: int = 148, candidates=(768, 1024, 1280, 1536, 1792, 2048)) -> int:
    """Tokens per CTA for a batch with these context lengths: the candidate whose launch the model above finishes first. How the
    chunks of a batch fall into waves of resident CTAs moves a launch by a few per cent, and which size is best depends on the
    lengths; the choice is made where a step is captured (lengths grow by one token per step, so it holds for many steps)."""
    ctx = [int(c) for c in ctx_lens]
    if not ctx or kv_heads <= 0:
        return 1024
    return min(candidates, key=lambda c: (simulate_decode_launch(ctx, kv_heads, c, slots=2 * sms), c))


class PagedAttention:
    """Holds the split-KV scratch (partials, statistics, counters) for a maximum batch and context."""

    def __init__(self, device, max_batch: int, q_heads: int, kv_heads: int, max_ctx: int, chunk_tokens: int = 512, impl: str = "simt"):
        """impl: "tc" (tcgen05 tensor cores, one CTA per (sequence, split, KV head); chunk_tokens % 128 == 0) or "simt" (CUDA
        cores, paged_attn.cu: the second implementation and the oracle of the first)."""
        assert impl in ("simt", "tc") and (impl == "simt" or chunk_tokens % 128 == 0)
        self.impl = impl
        self._C = load()
        self.device = torch.device(device)
        self.q_heads, self.kv_heads, self.chunk_tokens, self.max_ctx = q_heads, kv_heads, chunk_tokens, max_ctx
        self.max_splits = (max_ctx + chunk_tokens - 1) // chunk_tokens
        self.part_o = torch.empty((max_batch, q_heads, self.max_splits, 128), dtype=torch.float32, device=self.device)
        self.part_m = torch.empty((max_batch, q_heads, self.max_splits), dtype=torch.float32, device=self.device)
        self.part_l = torch.empty_like(self.part_m)
        self.counters = torch.zeros((max_batch * kv_heads,), dtype=torch.int32, device=self.device)
        self.status = new_status(self.device)
        self.max_batch = max_batch

    def __call__(self, q: torch.Tensor, pool: PagedKVPool, layer: int, block_table: torch.Tensor, ctx_lens: torch.Tensor,
                 max_ctx: Optional[int] = None, out: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
        assert pool.layout == "hnd" and q.shape[0] <= self.max_batch and q.shape[1] == self.q_heads
        if out is None:
            out = torch.empty_like(q)
        bs, ls, ks = pool.strides
        self._C.paged_attn_decode(q, pool.layer_base(layer), out, block_table, ctx_lens, bs, ks, pool.head_stride, self.kv_heads,
                                  min(max_ctx or self.max_ctx, self.max_ctx, block_table.shape[1] * 16), self.chunk_tokens,
                                  scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]),
                                  self.part_o, self.part_m, self.part_l, self.counters, self.status,
                                  (pool.data.numel() - layer * ls) // 128 if self.impl != "simt" else 0,
                                  num_blocks=pool.data.shape[0])
        return out


class PrefillAttention:
    """Causal attention of prompts, or of the next piece of each prompt, against their K/V in the paged pool
    (prefill_attn_tc.cu): tcgen05 MMAs with the accumulators in TMEM, K/V pages fetched by TMA straight from the pool in
    either layout, two 128-token query tiles per CTA. Pages must hold finite values past a prompt's last token (a fresh
    pool is zeroed); block-table entries past a prompt's pages must name valid blocks."""

    def __init__(self, device):
        self._C = load()
        self.device = torch.device(device)
        self.status = new_status(self.device)

    def __call__(self, q: torch.Tensor, pool: PagedKVPool, layer: int, block_table: torch.Tensor, seq_start: torch.Tensor, max_len: int,
                 out: Optional[torch.Tensor] = None, scale: Optional[float] = None, pos0: Optional[torch.Tensor] = None) -> torch.Tensor:
        """q: [tokens][q_heads][128] with the prompts (or pieces of prompts) packed back to back; seq_start: int32
        [n_seqs + 1] token offsets into q; max_len: the longest piece. pos0 (int32 [n_seqs], optional): how many tokens of
        each sequence precede its first query here; their K/V are already in the pool and every query attends to them
        (chunked prefill). Without it every sequence starts at position 0."""
        if out is None:
            out = torch.empty_like(q)
        bs, ls, ks = pool.strides
        g = pool.geom
        if pool.layout == "hnd":
            head_stride, tok_stride = g.block_tokens * g.head_dim, g.head_dim
        else:
            head_stride, tok_stride = g.head_dim, g.kv_heads * g.head_dim
        self._C.prefill_attn(q, pool.layer_base(layer), out, block_table, seq_start, bs, ks, head_stride, tok_stride, g.kv_heads, int(max_len),
                             scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]), self.status,
                             (pool.data.numel() - layer * ls) // 128, pos0)
        return out


def prefill_attn_reference(q: torch.Tensor, pool: PagedKVPool, layer: int, block_table: torch.Tensor, seq_lens, scale: Optional[float] = None,
                           pos0=None) -> torch.Tensor:
    """Plain fp32 causal softmax attention of packed prompts over the gathered pages (test oracle). ``seq_lens``: queries per
    sequence in ``q``; ``pos0``: tokens of each sequence that precede them (already in the pool), default none."""
    T, Hq, D = q.shape
    Hkv = pool.geom.kv_heads
    G = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty((T, Hq, D), dtype=torch.float32, device=q.device)
    o = 0
    for s, n in enumerate(seq_lens):
        n = int(n)
        p0 = int(pos0[s]) if pos0 is not None else 0
        nk = p0 + n
        nb = (nk + 15) // 16
        kv = pool.data[block_table[s, :nb].long(), layer]
        if pool.layout == "nhd":
            kv = kv.permute(0, 1, 3, 2, 4)                 # -> [nb][2][H][16][D]
        k = kv[:, 0].permute(1, 0, 2, 3).reshape(Hkv, nb * 16, D)[:, :nk].float()
        v = kv[:, 1].permute(1, 0, 2, 3).reshape(Hkv, nb * 16, D)[:, :nk].float()
        qs = q[o:o + n].float().view(n, Hkv, G, D).permute(1, 2, 0, 3)          # [Hkv][G][n][D]
        sc = torch.einsum("hgqd,hkd->hgqk", qs, k) * scale
        mask = torch.ones((n, nk), dtype=torch.bool, device=q.device).tril(diagonal=p0)     # query i sees keys 0 .. p0 + i
        sc = sc.masked_fill(~mask, float("-inf"))
        pr = torch.softmax(sc, dim=-1)
        out[o:o + n] = torch.einsum("hgqk,hkd->hgqd", pr, v).permute(2, 0, 1, 3).reshape(n, Hq, D)
        o += n
    return out


def paged_attn_reference(q: torch.Tensor, pool: PagedKVPool, layer: int, block_table: torch.Tensor, ctx_lens: torch.Tensor,
                         scale: Optional[float] = None) -> torch.Tensor:
    """Plain fp32 softmax attention over the gathered pages (test oracle)."""
    B, Hq, D = q.shape
    Hkv = pool.geom.kv_heads
    G = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty((B, Hq, D), dtype=torch.float32, device=q.device)
    for b in range(B):
        n = int(ctx_lens[b])
        nb = (n + 15) // 16
        blocks = block_table[b, :nb].long()
        kv = pool.data[blocks, layer]                      # hnd: [nb][2][H][16][D]
        if pool.layout == "nhd":
            kv = kv.permute(0, 1, 3, 2, 4)
        k = kv[:, 0].permute(1, 0, 2, 3).reshape(Hkv, nb * 16, D)[:, :n].float()
        v = kv[:, 1].permute(1, 0, 2, 3).reshape(Hkv, nb * 16, D)[:, :n].float()
        qb = q[b].float().view(Hkv, G, D)
        s = torch.einsum("hgd,htd->hgt", qb, k) * scale
        p = torch.softmax(s, dim=-1)
        out[b] = torch.einsum("hgt,htd->hgd", p, v).reshape(Hq, D)
    return out
