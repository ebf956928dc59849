"""Comparison arm for the fused tensor-parallel kernels: the same decoder step with library collectives and GEMMs.

all-gather and reduce-scatter are torch.distributed calls (NCCL over NVLink), GEMMs are torch.matmul (cuBLAS);
norms, RoPE + KV append, paged attention, SiLU*mul and sampling stay this package's kernels, so the difference to
``TPDecoder`` is exactly what this package's GEMMs and the collectives fused into them buy. This is the baseline
mechanism (a library call per collective and per GEMM), not the product path. With one rank there is no collective
and the arm is the decoder on cuBLAS GEMMs.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..models.qwen3 import Qwen3Decoder


class NcclTPDecoder:
    def __init__(self, cfg, weights, pool, batch, max_ctx, rank, world, attn, group=None, collective: str = "rs_ag", fp32_matmul: bool = False):
        """collective: "rs_ag" = reduce-scatter + all-gather around a token-sharded residual stream (four library collectives per
        layer); "allreduce" = one all-reduce after each row-parallel GEMM with the residual stream replicated (two per layer, the
        form inference servers use for decode).
        fp32_matmul: every GEMM as torch.matmul on fp32 copies of the same bf16 operands, the result rounded to bf16 where the
        bf16 GEMM rounds it. Products of bf16 numbers are exact in fp32, so this differs from the bf16 GEMM only in the order of
        the fp32 sums: a third implementation with the same rounding points, used to measure how far two correct implementations
        drift apart over the layers. Slow; for checks, not for timing."""
        assert collective in ("rs_ag", "allreduce")
        self.collective = collective
        self.fp32_matmul = fp32_matmul
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
        self.logits = None                      # this rank's vocabulary slice of the last step's logits
        if collective == "allreduce":
            self.resid_full = torch.zeros((batch, H), **bf)
            self.xn_full = torch.empty((batch, H), **bf)

    def _all_gather(self, out, x):
        if self.world > 1:
            dist.all_gather_into_tensor(out, x, group=self.group)
        else:
            out.copy_(x)

    def _reduce_scatter(self, out, x):
        if self.world > 1:
            dist.reduce_scatter_tensor(out, x, group=self.group)
        else:
            out.copy_(x)

    def _mm(self, x, w, out=None):
        """x @ w^T in bf16 (cuBLAS), or with fp32_matmul on fp32 copies."""
        if not self.fp32_matmul:
            return torch.matmul(x, w.t(), out=out) if out is not None else torch.matmul(x, w.t())
        r = torch.matmul(x.float(), w.float().t()).to(torch.bfloat16)
        if out is not None:
            out.copy_(r)
            return out
        return r

    @classmethod
    def from_engine(cls, eng, collective: str = "rs_ag", fp32_matmul: bool = False) -> "NcclTPDecoder":
        b = cls(eng.cfg, eng.w, eng.pool, eng.max_batch, eng.max_ctx, getattr(eng, "rank", 0), getattr(eng, "world", 1), eng.attn,
                collective=collective, fp32_matmul=fp32_matmul)
        b.ids.copy_(eng.ids); b.positions.copy_(eng.positions); b.ctx_lens.copy_(eng.ctx_lens)
        b.block_table = eng.block_table
        return b

    def _pick(self, x_full) -> None:
        """lm_head on this rank's vocabulary slice, then the global argmax through two all-gathers."""
        w = self.w
        logits = self.logits = self._mm(x_full, w.lm_head)
        val, idx = logits.float().max(-1)
        self._all_gather(self.max_val.view(-1), val)
        self._all_gather(self.max_idx.view(-1), idx + w.vocab_lo)
        best = self.max_val.argmax(0)
        self.next_ids.copy_(self.max_idx.gather(0, best[None])[0].int())

    def _step_allreduce(self, b: int, max_ctx: int) -> None:
        cfg, w = self.cfg, self.w
        resid, xn, part = self.resid_full, self.xn_full, self.partial
        ops.embedding(self.ids, w.embed, out=resid)
        for li, lw in enumerate(w.layers):
            if li == 0:
                ops.rmsnorm(resid, lw.ln1, cfg.eps, out=xn)
            else:
                ops.rmsnorm(part, lw.ln1, cfg.eps, residual=resid, out=xn)
            qkv = self._mm(xn, lw.qkv)
            ops.rope_append(qkv, lw.q_norm, lw.k_norm, self.pool, li, self.inv_freq, self.block_table, self.positions, self.qh, cfg.eps, q_out=self.q)
            self.attn(self.q, self.pool, li, self.block_table, self.ctx_lens, max_ctx=max_ctx, out=self.attn_out)
            self._mm(self.attn_out.view(b, -1), lw.o, out=part)
            if self.world > 1:
                dist.all_reduce(part, group=self.group)
            ops.rmsnorm(part, lw.ln2, cfg.eps, residual=resid, out=xn)
            act = ops.silu_mul(self._mm(xn, lw.gate_up))
            self._mm(act, lw.down, out=part)
            if self.world > 1:
                dist.all_reduce(part, group=self.group)
        ops.rmsnorm(part, w.final_norm, cfg.eps, residual=resid, out=xn)
        self._pick(xn)

    def _step(self, b: int, max_ctx: int) -> None:
        if self.collective == "allreduce":
            return self._step_allreduce(b, max_ctx)
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
            self._all_gather(self.x_full, self.xn_local)
            qkv = self._mm(self.x_full, lw.qkv)
            ops.rope_append(qkv, lw.q_norm, lw.k_norm, self.pool, li, self.inv_freq, self.block_table, self.positions, self.qh, cfg.eps, q_out=self.q)
            self.attn(self.q, self.pool, li, self.block_table, self.ctx_lens, max_ctx=max_ctx, out=self.attn_out)
            self._mm(self.attn_out.view(b, -1), lw.o, out=self.partial)
            self._reduce_scatter(self.h_local, self.partial)
            ops.rmsnorm(self.h_local, lw.ln2, cfg.eps, residual=self.resid, out=self.xn_local)
            self._all_gather(self.x_full, self.xn_local)
            gu = self._mm(self.x_full, lw.gate_up)
            act = ops.silu_mul(gu)
            self._mm(act, lw.down, out=self.partial)
            self._reduce_scatter(self.h_local, self.partial)
        ops.rmsnorm(self.h_local, w.final_norm, cfg.eps, residual=self.resid, out=self.xn_local)
        self._all_gather(self.x_full, self.xn_local)
        self._pick(self.x_full)

    _advance = Qwen3Decoder._advance
    step = Qwen3Decoder.step
    capture = Qwen3Decoder.capture
    replay = Qwen3Decoder.replay

    def check_status(self) -> str:
        torch.cuda.synchronize(self.device)
        return "OK"
