"""Qwen3 dense decoder on the sm_100a kernels: random-init weights, paged KV
cache, decode engine (optionally captured in a CUDA graph) and a prefill path.

Architecture (Qwen3-8B): 36 layers, hidden 4096, 32 query / 8 KV heads of 128,
SwiGLU FFN 12288, vocabulary 151936, RMSNorm, per-head QK-norm, rotary
embedding (theta 1e6), untied lm_head.

The reference does not contain a model: its decode workloads are KV-scan
stressors (llm_problem_analysis/decode_vllm_kvcache_hbm_stress.cu,
llm_problem_analysis/decode_transformer_kvcache_stress.cu) and its README names
Qwen3-8B under vLLM as the case study (README.md:56-75). This is that decoder,
built on this package's own kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import ops
from ..ops.kv_cache import KVGeometry, PagedKVPool


@dataclass
class Qwen3Config:
    layers: int = 36
    hidden: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 12288
    vocab: int = 151936
    rope_theta: float = 1e6
    eps: float = 1e-6
    name: str = "qwen3-8b"

    @classmethod
    def tiny(cls, layers: int = 2, vocab: int = 1024) -> "Qwen3Config":
        return cls(layers=layers, hidden=512, q_heads=8, kv_heads=2, ffn=1024, vocab=vocab, name="qwen3-tiny")

    @classmethod
    def from_hf(cls, hf) -> "Qwen3Config":
        """From a Hugging Face ``Qwen3Config`` (or anything with the same attribute names)."""
        rope = getattr(hf, "rope_theta", None)
        if rope is None:                                    # newer configs keep it inside rope_parameters
            rope = (getattr(hf, "rope_parameters", None) or {}).get("rope_theta", 1e6)
        return cls(layers=hf.num_hidden_layers, hidden=hf.hidden_size, q_heads=hf.num_attention_heads, kv_heads=hf.num_key_value_heads,
                   head_dim=getattr(hf, "head_dim", None) or hf.hidden_size // hf.num_attention_heads, ffn=hf.intermediate_size,
                   vocab=hf.vocab_size, rope_theta=float(rope), eps=float(hf.rms_norm_eps), name=getattr(hf, "name_or_path", "") or "qwen3")

    @property
    def geometry(self) -> KVGeometry:
        return KVGeometry(self.layers, self.kv_heads, self.head_dim)

    def param_count(self) -> int:
        per_layer = (self.q_heads + 2 * self.kv_heads) * self.head_dim * self.hidden + self.q_heads * self.head_dim * self.hidden \
            + 3 * self.ffn * self.hidden + 2 * self.hidden + 2 * self.head_dim
        return self.layers * per_layer + 2 * self.vocab * self.hidden + self.hidden


class LayerWeights:
    __slots__ = ("qkv", "o", "gate_up", "down", "ln1", "ln2", "q_norm", "k_norm")


class Qwen3Weights:
    """Random-init weights in the fused layouts the kernels take: qkv rows = [q heads | k heads | v heads],
    gate_up rows = [gate | up]. ``shard(rank, world)`` returns the tensor-parallel slice."""

    def __init__(self, cfg: Qwen3Config, device="cuda", seed: int = 0, std: float = 0.02, tp_rank: int = 0, tp_world: int = 1):
        self.cfg, self.tp_rank, self.tp_world = cfg, tp_rank, tp_world
        gen = torch.Generator(device=device)
        H, D = cfg.hidden, cfg.head_dim
        assert cfg.q_heads % tp_world == 0 and cfg.kv_heads % tp_world == 0 and cfg.ffn % tp_world == 0
        qh, kh, ff = cfg.q_heads // tp_world, cfg.kv_heads // tp_world, cfg.ffn // tp_world

        def rnd(rows, cols, tag, scale=std):
            # every (tensor, rank) draws from its own stream, so a shard equals the same rows of the full tensor
            gen.manual_seed(seed * 1000003 + tag)
            return (torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * scale).to(torch.bfloat16)

        def rows_of(full_rows, tag, lo, hi, cols, scale=std):
            full = rnd(full_rows, cols, tag, scale)
            return full[lo:hi].contiguous()

        self.layers: List[LayerWeights] = []
        for li in range(cfg.layers):
            w = LayerWeights()
            t = li * 16
            q = rows_of(cfg.q_heads * D, t + 1, tp_rank * qh * D, (tp_rank + 1) * qh * D, H)
            k = rows_of(cfg.kv_heads * D, t + 2, tp_rank * kh * D, (tp_rank + 1) * kh * D, H)
            v = rows_of(cfg.kv_heads * D, t + 3, tp_rank * kh * D, (tp_rank + 1) * kh * D, H)
            w.qkv = torch.cat([q, k, v], 0).contiguous()
            o_full = rnd(H, cfg.q_heads * D, t + 4)
            w.o = o_full[:, tp_rank * qh * D:(tp_rank + 1) * qh * D].contiguous()       # row-parallel: K is sharded
            gate = rows_of(cfg.ffn, t + 5, tp_rank * ff, (tp_rank + 1) * ff, H)
            up = rows_of(cfg.ffn, t + 6, tp_rank * ff, (tp_rank + 1) * ff, H)
            w.gate_up = torch.cat([gate, up], 0).contiguous()
            down_full = rnd(H, cfg.ffn, t + 7)
            w.down = down_full[:, tp_rank * ff:(tp_rank + 1) * ff].contiguous()
            del o_full, down_full
            gen.manual_seed(seed * 1000003 + t + 8)
            w.ln1 = (1.0 + 0.1 * torch.randn(H, generator=gen, device=device)).to(torch.bfloat16)
            w.ln2 = (1.0 + 0.1 * torch.randn(H, generator=gen, device=device)).to(torch.bfloat16)
            w.q_norm = (1.0 + 0.1 * torch.randn(D, generator=gen, device=device)).to(torch.bfloat16)
            w.k_norm = (1.0 + 0.1 * torch.randn(D, generator=gen, device=device)).to(torch.bfloat16)
            self.layers.append(w)
        self.embed = rnd(cfg.vocab, H, 900001, 1.0)
        vs = (cfg.vocab + tp_world - 1) // tp_world
        self.vocab_lo, self.vocab_hi = tp_rank * vs, min(cfg.vocab, (tp_rank + 1) * vs)
        self.lm_head = rows_of(cfg.vocab, 900002, self.vocab_lo, self.vocab_hi, H)
        gen.manual_seed(seed * 1000003 + 900003)
        self.final_norm = (1.0 + 0.1 * torch.randn(H, generator=gen, device=device)).to(torch.bfloat16)

    @classmethod
    def from_state_dict(cls, cfg: Qwen3Config, sd, device="cuda", tp_rank: int = 0, tp_world: int = 1) -> "Qwen3Weights":
        """Weights from a checkpoint in the Hugging Face Qwen3 naming (``model.layers.N.self_attn.q_proj.weight`` ...,
        a ``state_dict()`` or any mapping of name -> tensor), converted to bf16 in the fused layouts the kernels take and cut
        to the tensor-parallel shard ``tp_rank`` of ``tp_world``: qkv rows = this rank's [q heads | k heads | v heads], gate_up
        rows = [gate | up] columns of this rank, O and down as the matching input slices, lm_head as a vocabulary slice.
        With tied embeddings (no ``lm_head.weight``) the embedding table is the output projection."""
        self = cls.__new__(cls)
        self.cfg, self.tp_rank, self.tp_world = cfg, tp_rank, tp_world
        H, D = cfg.hidden, cfg.head_dim
        assert cfg.q_heads % tp_world == 0 and cfg.kv_heads % tp_world == 0 and cfg.ffn % tp_world == 0
        qh, kh, ff = cfg.q_heads // tp_world, cfg.kv_heads // tp_world, cfg.ffn // tp_world

        def t(name, shape):
            x = sd[name]
            assert tuple(x.shape) == tuple(shape), (name, tuple(x.shape), tuple(shape))
            return x.detach().to(device=device, dtype=torch.bfloat16)

        self.layers = []
        for li in range(cfg.layers):
            pre = f"model.layers.{li}."
            w = LayerWeights()
            q = t(pre + "self_attn.q_proj.weight", (cfg.q_heads * D, H))[tp_rank * qh * D:(tp_rank + 1) * qh * D]
            k = t(pre + "self_attn.k_proj.weight", (cfg.kv_heads * D, H))[tp_rank * kh * D:(tp_rank + 1) * kh * D]
            v = t(pre + "self_attn.v_proj.weight", (cfg.kv_heads * D, H))[tp_rank * kh * D:(tp_rank + 1) * kh * D]
            w.qkv = torch.cat([q, k, v], 0).contiguous()
            w.o = t(pre + "self_attn.o_proj.weight", (H, cfg.q_heads * D))[:, tp_rank * qh * D:(tp_rank + 1) * qh * D].contiguous()
            gate = t(pre + "mlp.gate_proj.weight", (cfg.ffn, H))[tp_rank * ff:(tp_rank + 1) * ff]
            up = t(pre + "mlp.up_proj.weight", (cfg.ffn, H))[tp_rank * ff:(tp_rank + 1) * ff]
            w.gate_up = torch.cat([gate, up], 0).contiguous()
            w.down = t(pre + "mlp.down_proj.weight", (H, cfg.ffn))[:, tp_rank * ff:(tp_rank + 1) * ff].contiguous()
            w.ln1 = t(pre + "input_layernorm.weight", (H,)).clone()
            w.ln2 = t(pre + "post_attention_layernorm.weight", (H,)).clone()
            w.q_norm = t(pre + "self_attn.q_norm.weight", (D,)).clone()
            w.k_norm = t(pre + "self_attn.k_norm.weight", (D,)).clone()
            self.layers.append(w)
        self.embed = t("model.embed_tokens.weight", (cfg.vocab, H)).contiguous()
        vs = (cfg.vocab + tp_world - 1) // tp_world
        self.vocab_lo, self.vocab_hi = tp_rank * vs, min(cfg.vocab, (tp_rank + 1) * vs)
        head = t("lm_head.weight", (cfg.vocab, H)) if "lm_head.weight" in sd else self.embed
        self.lm_head = head[self.vocab_lo:self.vocab_hi].clone().contiguous()
        self.final_norm = t("model.norm.weight", (H,)).clone()
        return self

    def nbytes(self) -> int:
        n = self.embed.numel() + self.lm_head.numel() + self.final_norm.numel()
        for w in self.layers:
            n += sum(getattr(w, k).numel() for k in LayerWeights.__slots__)
        return n * 2


class Qwen3Decoder:
    """Single-GPU decode engine: fixed-capacity batch, preallocated activations, optional CUDA graph."""

    def __init__(self, cfg: Qwen3Config, weights: Qwen3Weights, pool: PagedKVPool, max_batch: int, max_ctx: int,
                 attn_chunk: int = 1024, attn_impl: str = "tc", prefill_attn: str = "tc"):
        assert pool.layout == "hnd" and prefill_attn in ("tc", "sdpa")
        self.cfg, self.w, self.pool = cfg, weights, pool
        self.prefill_attn = prefill_attn              # default of prefill(): this package's kernel or the library arm
        # decode sampling: 0 = greedy (argmax); > 0 draws from softmax(logits / temperature), noise keyed by (sample_seed, position).
        # Set before capture(): a captured graph keeps the choice it was captured with.
        self.temperature, self.sample_seed = 0.0, 0
        self._prefill_attn = None
        dev = pool.data.device
        self.device = dev
        self.max_batch, self.max_ctx = max_batch, max_ctx
        B, H = max_batch, cfg.hidden
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.resid = torch.zeros((B, H), **bf)
        self.xn = torch.empty((B, H), **bf)
        self.h = torch.empty((B, H), **bf)
        self.qkv = torch.empty((B, (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim), **bf)
        self.q = torch.empty((B, cfg.q_heads, cfg.head_dim), **bf)
        self.attn_out = torch.empty((B, cfg.q_heads, cfg.head_dim), **bf)
        self.act = torch.empty((B, cfg.ffn), **bf)
        self.logits = torch.empty((B, weights.lm_head.shape[0]), **bf)
        self.next_ids = torch.zeros((B,), dtype=torch.int32, device=dev)
        self.ids = torch.zeros((B,), dtype=torch.int32, device=dev)
        self.positions = torch.zeros((B,), dtype=torch.int32, device=dev)
        self.ctx_lens = torch.ones((B,), dtype=torch.int32, device=dev)
        self.max_blocks = (max_ctx + 15) // 16
        self.block_table = torch.zeros((B, self.max_blocks), dtype=torch.int32, device=dev)
        self.inv_freq = ops.rope_inv_freq(cfg.rope_theta, dev, cfg.head_dim)
        self.attn = ops.PagedAttention(dev, B, cfg.q_heads, cfg.kv_heads, max_ctx, attn_chunk, impl=attn_impl)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.graph_batch = 0
        self.kernels_per_step = 1 + 8 * cfg.layers + 3   # embedding, 8 per layer, final norm, lm_head, argmax

    # ---- state ----
    def set_batch(self, ids: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor) -> None:
        """ids/positions: the token to feed for every sequence and its position; the cache already holds
        positions [0, position) of each sequence in the blocks of ``block_table``."""
        b = ids.numel()
        self.ids[:b].copy_(ids)
        self.positions[:b].copy_(positions)
        self.ctx_lens[:b].copy_(positions + 1)
        self.block_table[:b, :block_table.shape[1]].copy_(block_table)

    # ---- one decode step for the first `b` slots ----
    def _step(self, b: int, max_ctx: int) -> None:
        cfg, w = self.cfg, self.w
        resid, xn, h = self.resid[:b], self.xn[:b], self.h[:b]
        qkv, q, ao, act = self.qkv[:b], self.q[:b], self.attn_out[:b], self.act[:b]
        pos, ctx, table = self.positions[:b], self.ctx_lens[:b], self.block_table[:b]
        ops.embedding(self.ids[:b], w.embed, out=resid)
        for li, lw in enumerate(w.layers):
            if li == 0:
                ops.rmsnorm(resid, lw.ln1, cfg.eps, out=xn)
            else:
                ops.rmsnorm(h, lw.ln1, cfg.eps, residual=resid, out=xn)
            ops.gemm(xn, lw.qkv, out=qkv)
            ops.rope_append(qkv, lw.q_norm, lw.k_norm, self.pool, li, self.inv_freq, table, pos, cfg.q_heads, cfg.eps, q_out=q)
            self.attn(q, self.pool, li, table, ctx, max_ctx=max_ctx, out=ao)
            ops.gemm(ao.view(b, -1), lw.o, out=h)
            ops.rmsnorm(h, lw.ln2, cfg.eps, residual=resid, out=xn)
            ops.gemm(xn, lw.gate_up, out=act, gated=True)
            ops.gemm(act, lw.down, out=h)
        ops.rmsnorm(h, w.final_norm, cfg.eps, residual=resid, out=xn)
        ops.gemm(xn, w.lm_head, out=self.logits[:b])
        self._pick(b)

    def _pick(self, b: int) -> None:
        if self.temperature > 0:
            ops.sample(self.logits[:b], self.temperature, self.sample_seed, positions=self.positions[:b], out=self.next_ids[:b])
        else:
            ops.argmax(self.logits[:b], out=self.next_ids[:b])

    def _advance(self, b: int) -> None:
        self.ids[:b].copy_(self.next_ids[:b])
        self.positions[:b].add_(1)
        self.ctx_lens[:b].add_(1)

    def step(self, b: Optional[int] = None, max_ctx: Optional[int] = None, advance: bool = True) -> torch.Tensor:
        """Eager decode step. Returns the sampled ids (a view; valid until the next step)."""
        b = b or self.max_batch
        self._step(b, max_ctx or self.max_ctx)
        if advance:
            self._advance(b)
        return self.next_ids[:b]

    def capture(self, b: Optional[int] = None, max_ctx: Optional[int] = None) -> None:
        """Captures step+advance for batch ``b`` into a CUDA graph (launch-bound otherwise: ~290 kernels/step)."""
        b = b or self.max_batch
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        keep = (self.ids.clone(), self.positions.clone(), self.ctx_lens.clone())
        with torch.cuda.stream(s):
            self._step(b, max_ctx or self.max_ctx)      # warm-up outside capture (lazy attribute set-up, workspaces)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                self._step(b, max_ctx or self.max_ctx)
                self._advance(b)
        torch.cuda.current_stream(self.device).wait_stream(s)
        self.ids.copy_(keep[0]); self.positions.copy_(keep[1]); self.ctx_lens.copy_(keep[2])
        self.graph, self.graph_batch = g, b

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.next_ids[:self.graph_batch]

    def check_status(self) -> str:
        """"OK", or the first non-OK status a kernel of this engine left behind (bounded waits that gave up)."""
        from ..ops.flow import read_status
        from ..ops.gemm import workspace_for

        torch.cuda.synchronize(self.device)
        for st in (read_status(self.attn.status), read_status(workspace_for(self.device).status)):
            if st["status"] != 0:
                return f"{st['status_name']}:{st['detail']}"
        return "OK"

    def bytes_per_step(self, ctx: torch.Tensor) -> int:
        """HBM bytes one decode step must read on this GPU: the weights (the embedding table only by row) and the KV of ``ctx``."""
        weights = self.w.nbytes() - self.w.embed.numel() * 2 + self.max_batch * self.cfg.hidden * 2
        kv = int(ctx.sum()) * self.cfg.layers * 2 * self.pool.geom.kv_heads * self.cfg.head_dim * 2
        return weights + kv

    # ---- prefill: whole prompts, token-major or head-major pool, returns last-position logits ----
    @staticmethod
    def prefill_plan(seq_lens: List[int], chunk: int) -> List[List[tuple]]:
        """Cuts the prompts into passes of at most ``chunk`` tokens: a list of passes, each a list of (sequence, first token,
        end token). A prompt longer than the room left in a pass continues in the next one, so a sequence appears at most
        once per pass and its pieces run in order."""
        assert chunk >= 1
        passes, cur, room = [], [], chunk
        for s, n in enumerate(seq_lens):
            p = 0
            while p < n:
                take = min(n - p, room)
                cur.append((s, p, p + take))
                p += take
                room -= take
                if room == 0:
                    passes.append(cur)
                    cur, room = [], chunk
        if cur:
            passes.append(cur)
        return passes

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, seq_lens: List[int], block_table: torch.Tensor, pool: Optional[PagedKVPool] = None,
                chunk: int = 8192, attn: Optional[str] = None) -> torch.Tensor:
        """Runs the prompts through the stack, writing K/V into ``pool`` (default: the decode pool); returns the logits of
        every prompt's last position, [n_seqs][vocab].

        At most ``chunk`` tokens go through the stack at once, so the activations stay bounded whatever the prompt lengths: a
        long prompt is processed in pieces, each piece attending to the K/V that the earlier pieces left in the pool.
        GEMMs and K/V append use this package's kernels. The causal attention is this package's tcgen05 kernel reading the
        pages in place (``attn="tc"``, csrc/kernels/prefill_attn_tc.cu) or torch's scaled_dot_product_attention over gathered
        copies of K and V (``attn="sdpa"``, a library kernel, kept as the comparison arm). Default: ``self.prefill_attn``."""
        attn = attn or self.prefill_attn
        assert attn in ("tc", "sdpa")
        cfg, w = self.cfg, self.w
        pool = pool or self.pool
        dev = ids.device
        D = cfg.head_dim
        starts = [0]
        for n in seq_lens[:-1]:
            starts.append(starts[-1] + int(n))
        if attn == "tc" and self._prefill_attn is None:
            self._prefill_attn = ops.PrefillAttention(dev)
        last_hidden = [None] * len(seq_lens)
        for pieces in self.prefill_plan([int(n) for n in seq_lens], int(chunk)):
            lens = [e - b for _, b, e in pieces]
            T = sum(lens)
            tok = torch.cat([torch.arange(starts[s] + b, starts[s] + e, device=dev) for s, b, e in pieces])
            positions = torch.cat([torch.arange(b, e, device=dev) for _, b, e in pieces]).int()
            seq_ids = torch.repeat_interleave(torch.tensor([s for s, _, _ in pieces], device=dev, dtype=torch.int32),
                                              torch.tensor(lens, device=dev))
            seq_start = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32, device=dev)
            pos0 = torch.tensor([b for _, b, _ in pieces], dtype=torch.int32, device=dev)
            rows = block_table[torch.tensor([s for s, _, _ in pieces], device=block_table.device)].contiguous()
            resid = ops.embedding(ids[tok].int(), w.embed)
            h = None
            for li, lw in enumerate(w.layers):
                xn = ops.rmsnorm(resid, lw.ln1, cfg.eps) if h is None else ops.rmsnorm(h, lw.ln1, cfg.eps, residual=resid)
                qkv = ops.gemm(xn, lw.qkv)
                q = ops.rope_append(qkv, lw.q_norm, lw.k_norm, pool, li, self.inv_freq, block_table, positions, cfg.q_heads, cfg.eps,
                                    seq_ids=seq_ids)
                ao = torch.empty_like(q)
                if attn == "tc":
                    self._prefill_attn(q, pool, li, rows, seq_start, max(lens), out=ao, pos0=pos0)
                else:
                    o = 0
                    for (s, b, e), n in zip(pieces, lens):
                        nb = (e + 15) // 16
                        kvb = pool.data[block_table[s, :nb].long(), li]        # [nb][2][...]
                        if pool.layout == "hnd":
                            k = kvb[:, 0].permute(1, 0, 2, 3).reshape(cfg.kv_heads, nb * 16, D)[:, :e]
                            v = kvb[:, 1].permute(1, 0, 2, 3).reshape(cfg.kv_heads, nb * 16, D)[:, :e]
                        else:
                            k = kvb[:, 0].reshape(nb * 16, cfg.kv_heads, D)[:e].transpose(0, 1)
                            v = kvb[:, 1].reshape(nb * 16, cfg.kv_heads, D)[:e].transpose(0, 1)
                        qs = q[o:o + n].transpose(0, 1)                         # [Hq][n][D]
                        if b == 0:
                            out = torch.nn.functional.scaled_dot_product_attention(qs[None], k[None], v[None], is_causal=True, enable_gqa=True)
                        else:
                            mask = torch.ones((n, e), dtype=torch.bool, device=dev).tril(diagonal=b)
                            out = torch.nn.functional.scaled_dot_product_attention(qs[None], k[None], v[None], attn_mask=mask, enable_gqa=True)
                        ao[o:o + n] = out[0].transpose(0, 1)
                        o += n
                h = ops.gemm(ao.view(T, -1), lw.o)
                xn = ops.rmsnorm(h, lw.ln2, cfg.eps, residual=resid)
                act = ops.gemm(xn, lw.gate_up, gated=True)
                h = ops.gemm(act, lw.down)
            o = 0
            for (s, b, e), n in zip(pieces, lens):
                if e == int(seq_lens[s]):                                       # this piece ends its prompt: keep the last row
                    last_hidden[s] = (h[o + n - 1] if h is not None else torch.zeros_like(resid[0]), resid[o + n - 1])
                o += n
        hs = torch.stack([x[0] for x in last_hidden])
        rs = torch.stack([x[1] for x in last_hidden])
        xn = ops.rmsnorm(hs, w.final_norm, cfg.eps, residual=rs)
        return ops.gemm(xn, w.lm_head)


# ---------------------------------------------------------------------------
# Plain PyTorch reference of the same network (test oracle): fp32 math on the same bf16 weights,
# contiguous KV, no paging.

@torch.no_grad()
def reference_forward(cfg: Qwen3Config, w: Qwen3Weights, ids: torch.Tensor) -> torch.Tensor:
    """Full-sequence forward of one prompt; returns logits [tokens][vocab] in fp32."""
    T = ids.numel()
    D, Hq, Hkv = cfg.head_dim, cfg.q_heads, cfg.kv_heads

    def norm(x, g):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps) * g.float()

    def bf(x):
        return x.to(torch.bfloat16).float()

    inv = ops.rope_inv_freq(cfg.rope_theta, ids.device, D)
    pos = torch.arange(T, device=ids.device).float()
    ang = pos[:, None] * inv[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rope(x):
        x1, x2 = x[..., :D // 2], x[..., D // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    resid = w.embed[ids.long()].float()
    h = None
    for lw in w.layers:
        if h is not None:
            resid = bf(resid + h)
        xn = bf(norm(resid, lw.ln1))
        qkv = bf(xn @ lw.qkv.float().t()).view(T, Hq + 2 * Hkv, D)
        q = bf(rope(bf(norm(qkv[:, :Hq], lw.q_norm))))
        k = bf(rope(bf(norm(qkv[:, Hq:Hq + Hkv], lw.k_norm))))
        v = qkv[:, Hq + Hkv:]
        kr = k.repeat_interleave(Hq // Hkv, 1)
        vr = v.repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("thd,shd->hts", q, kr) / math.sqrt(D)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=ids.device), 1)[None], float("-inf"))
        ao = bf(torch.einsum("hts,shd->thd", torch.softmax(s, -1), vr)).reshape(T, Hq * D)
        h = bf(ao @ lw.o.float().t())
        resid = bf(resid + h)
        xn = bf(norm(resid, lw.ln2))
        gu = xn @ lw.gate_up.float().t()
        act = bf(torch.nn.functional.silu(gu[:, :cfg.ffn]) * gu[:, cfg.ffn:])
        h = bf(act @ lw.down.float().t())
    resid = bf(resid + h)
    xn = bf(norm(resid, w.final_norm))
    return xn @ w.lm_head.float().t()


def reference_forward_tp(cfg: Qwen3Config, w: Qwen3Weights, ids: torch.Tensor, group=None) -> torch.Tensor:
    """The same forward on a tensor-parallel shard of the weights (``Qwen3Weights(..., tp_rank, tp_world)``), in plain PyTorch
    with ``torch.distributed`` collectives, so it runs on CPU ranks over gloo: column-parallel QKV and gate/up (this rank's
    heads and FFN columns), row-parallel O and down whose bf16 partial products are summed over the ranks, and a
    vocabulary-parallel lm_head. Returns this rank's logits columns [tokens][vocab_hi - vocab_lo] in fp32. It states what
    ``parallel.TPDecoder`` must compute and checks the shard layout without a GPU."""
    import torch.distributed as dist

    world = w.tp_world
    T = ids.numel()
    D, Hq, Hkv, F = cfg.head_dim, cfg.q_heads // world, cfg.kv_heads // world, cfg.ffn // world

    def norm(x, g):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps) * g.float()

    def bf(x):
        return x.to(torch.bfloat16).float()

    def allsum(partial):
        x = bf(partial).contiguous()                 # each rank's partial tile travels as bf16
        if world > 1:
            dist.all_reduce(x, group=group)
        return bf(x)

    inv = ops.rope_inv_freq(cfg.rope_theta, ids.device, D)
    ang = torch.arange(T, device=ids.device).float()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rope(x):
        x1, x2 = x[..., :D // 2], x[..., D // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    resid = w.embed[ids.long()].float()
    h = None
    mask = torch.triu(torch.ones(T, T, dtype=torch.bool, device=ids.device), 1)[None]
    for lw in w.layers:
        if h is not None:
            resid = bf(resid + h)
        xn = bf(norm(resid, lw.ln1))
        qkv = bf(xn @ lw.qkv.float().t()).view(T, Hq + 2 * Hkv, D)
        q = bf(rope(bf(norm(qkv[:, :Hq], lw.q_norm))))
        k = bf(rope(bf(norm(qkv[:, Hq:Hq + Hkv], lw.k_norm))))
        v = qkv[:, Hq + Hkv:]
        kr, vr = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
        s = (torch.einsum("thd,shd->hts", q, kr) / math.sqrt(D)).masked_fill(mask, float("-inf"))
        ao = bf(torch.einsum("hts,shd->thd", torch.softmax(s, -1), vr)).reshape(T, Hq * D)
        h = allsum(ao @ lw.o.float().t())
        resid = bf(resid + h)
        xn = bf(norm(resid, lw.ln2))
        gu = xn @ lw.gate_up.float().t()
        act = bf(torch.nn.functional.silu(gu[:, :F]) * gu[:, F:])
        h = allsum(act @ lw.down.float().t())
    resid = bf(resid + h)
    xn = bf(norm(resid, w.final_norm))
    return xn @ w.lm_head.float().t()


class DecodeSession:
    """The call a user makes to decode: host token ids in, host token ids out, one step at a time.

    Every ``step`` copies the step's inputs (ids and positions, pinned host memory) to the device, runs the
    captured decode graph, and reads the sampled ids back to pinned host memory."""

    def __init__(self, engine: "Qwen3Decoder", batch: int, max_ctx: Optional[int] = None):
        self.eng, self.batch = engine, batch
        self.h_ids = torch.zeros(batch, dtype=torch.int32).pin_memory()
        self.h_pos = torch.zeros(batch, dtype=torch.int32).pin_memory()
        self.h_out = torch.zeros(batch, dtype=torch.int32).pin_memory()
        self.max_ctx = max_ctx or engine.max_ctx
        if engine.graph is None or engine.graph_batch != batch:
            engine.capture(batch, self.max_ctx)
        self.h2d_bytes_per_step = self.h_ids.numel() * 4 + self.h_pos.numel() * 4
        self.d2h_bytes_per_step = self.h_out.numel() * 4

    def start(self, ids: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor) -> None:
        self.eng.set_batch(ids.to(self.eng.device), positions.to(self.eng.device), block_table.to(self.eng.device))
        self.h_ids.copy_(ids.cpu())
        self.h_pos.copy_(positions.cpu())

    def step(self) -> torch.Tensor:
        e, b = self.eng, self.batch
        e.ids[:b].copy_(self.h_ids, non_blocking=True)
        e.positions[:b].copy_(self.h_pos, non_blocking=True)
        e.ctx_lens[:b].copy_(e.positions[:b])
        e.ctx_lens[:b].add_(1)
        e.replay()
        self.h_out.copy_(e.next_ids[:b], non_blocking=True)
        torch.cuda.current_stream(e.device).synchronize()
        self.h_ids.copy_(self.h_out)
        self.h_pos.add_(1)
        return self.h_out
