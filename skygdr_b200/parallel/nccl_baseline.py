"""Comparison arm for the fused tensor-parallel kernels: the same decoder step with library collectives and GEMMs.

all-gather and reduce-scatter are torch.distributed calls (NCCL over NVLink), GEMMs are torch.matmul (cuBLAS);
norms, RoPE + KV append, paged attention, SiLU*mul and sampling stay this package's kernels, so the difference to
``TPDecoder`` is exactly what fusing the collectives into the GEMM and norm kernels buys. This is the baseline
mechanism (a library call per collective), not the product path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..models.qwen3 import Qwen3Decoder


class NcclTPDecoder:
    def __init__(self, cfg, weights, pool, batch, max_ctx, rank, world, attn, group=None):
        self.cfg, self.w, self.pool, self.batch, self.max_ctx, self.rank, self.world, self.attn, self.group = \
            cfg, weights, pool, batch, max_ctx, rank, world, attn, group
        dev = pool.data.device
        self.device = dev
        self.rows = batch // world
        self.qh, self.kh = cfg.q_heads // world, cfg.kv_heads // world
        bf = dict(dtype=torch.bfloat16, device=dev)
        H = cfg.hidden
        self.resid = torch.zeros((self.rows, H), **bf)
        self.xn_local = torch.empty((self.rows, H), **bf)
        self.x_full = torch.empty((batch, H), **bf)
        self.partial = torch.empty((batch, H), **bf)
        self.h_local = torch.empty((self.rows, H), **bf)
        self.q = torch.empty((batch, self.qh, cfg.head_dim), **bf)
        self.attn_out = torch.empty((batch, self.qh, cfg.head_dim), **bf)
        self.max_val = torch.empty((world, batch), dtype=torch.float32, device=dev)
        self.max_idx = torch.empty((world, batch), dtype=torch.int64, device=dev)
        self.next_ids = torch.zeros((batch,), dtype=torch.int32, device=dev)
        self.ids = torch.zeros((batch,), dtype=torch.int32, device=dev)
        self.positions = torch.zeros((batch,), dtype=torch.int32, device=dev)
        self.ctx_lens = torch.ones((batch,), dtype=torch.int32, device=dev)
        self.block_table = None
        self.inv_freq = ops.rope_inv_freq(cfg.rope_theta, dev, cfg.head_dim)
        self.graph, self.graph_batch = None, batch
        self.max_batch = batch

    @classmethod
    def from_engine(cls, eng) -> "NcclTPDecoder":
        b = cls(eng.cfg, eng.w, eng.pool, eng.batch, eng.max_ctx, eng.rank, eng.world, eng.attn)
        b.ids.copy_(eng.ids); b.positions.copy_(eng.positions); b.ctx_lens.copy_(eng.ctx_lens)
        b.block_table = eng.block_table
        return b

    def _step(self, b: int, max_ctx: int) -> None:
        cfg, w = self.cfg, self.w
        r0 = self.rank * self.rows
        ops.embedding(self.ids[r0:r0 + self.rows], w.embed, out=self.resid)
        first = True
        for li, lw in enumerate(w.layers):
            if first:
                ops.rmsnorm(self.resid, lw.ln1, cfg.eps, out=self.xn_local)
                first = False
            else:
                ops.rmsnorm(self.h_local, lw.ln1, cfg.eps, residual=self.resid, out=self.xn_local)
            dist.all_gather_into_tensor(self.x_full, self.xn_local, group=self.group)
            qkv = torch.matmul(self.x_full, lw.qkv.t())
            ops.rope_append(qkv, lw.q_norm, lw.k_norm, self.pool, li, self.inv_freq, self.block_table, self.positions, self.qh, cfg.eps, q_out=self.q)
            self.attn(self.q, self.pool, li, self.block_table, self.ctx_lens, max_ctx=max_ctx, out=self.attn_out)
            torch.matmul(self.attn_out.view(b, -1), lw.o.t(), out=self.partial)
            dist.reduce_scatter_tensor(self.h_local, self.partial, group=self.group)
            ops.rmsnorm(self.h_local, lw.ln2, cfg.eps, residual=self.resid, out=self.xn_local)
            dist.all_gather_into_tensor(self.x_full, self.xn_local, group=self.group)
            gu = torch.matmul(self.x_full, lw.gate_up.t())
            act = ops.silu_mul(gu)
            torch.matmul(act, lw.down.t(), out=self.partial)
            dist.reduce_scatter_tensor(self.h_local, self.partial, group=self.group)
        ops.rmsnorm(self.h_local, w.final_norm, cfg.eps, residual=self.resid, out=self.xn_local)
        dist.all_gather_into_tensor(self.x_full, self.xn_local, group=self.group)
        logits = torch.matmul(self.x_full, w.lm_head.t())
        val, idx = logits.float().max(-1)
        dist.all_gather_into_tensor(self.max_val, val, group=self.group)
        dist.all_gather_into_tensor(self.max_idx, idx + w.vocab_lo, group=self.group)
        best = self.max_val.argmax(0)
        self.next_ids.copy_(self.max_idx.gather(0, best[None])[0].int())

    _advance = Qwen3Decoder._advance
    step = Qwen3Decoder.step
    capture = Qwen3Decoder.capture
    replay = Qwen3Decoder.replay

    def check_status(self) -> str:
        torch.cuda.synchronize(self.device)
        return "OK"
