"""Tensor-parallel Qwen3 decode over NVLink peer memory.

Megatron-style sharding: QKV / gate / up are column-parallel, O / down row-parallel, the residual
stream is sharded by token between blocks. The two collectives of each block are not library calls:

* all-gather -> GEMM: the norm kernel stores each normalised token row into every rank's gather
  buffer; the GEMM's TMA producer streams weights immediately and waits (bounded) for the rows.
* GEMM -> reduce-scatter: the GEMM epilogue stores each partial row into the owning rank's receive
  buffer; that rank's next norm kernel sums the partials, adds the residual and normalises.

Greedy sampling is vocabulary-parallel with the same push-and-count exchange. No NCCL call is on
the step path; NCCL only carries the one-time IPC handle exchange and barriers.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from .._ext import load
from ..models.qwen3 import Qwen3Config, Qwen3Decoder, Qwen3Weights
from ..ops.flow import new_status, read_status
from ..ops.gemm import FUSED_TP, GemmWorkspace, choose_config, pick_config
from ..ops.kv_cache import KVGeometry, PagedKVPool
from .symm import SymmetricHeap

TIMEOUT_NS = 2_000_000_000


class TPDecoder:
    def __init__(self, cfg: Qwen3Config, weights: Qwen3Weights, pool: PagedKVPool, batch: int, max_ctx: int, rank: int, world: int,
                 attn_chunk: int = 1024, group=None, attn_impl: str = "tc", collective: str = "oneshot"):
        """collective: "oneshot" = every rank pushes its full partial tile to every peer in the GEMM epilogue and the norm kernel
        sums `world` partials, with the residual stream and the normed activations replicated (2 hops per layer, world-1 times
        the bytes: decode tiles are small enough for that); "rs_ag" = GEMM -> reduce-scatter and all-gather -> GEMM with a
        token-sharded residual stream (4 hops per layer, the fewest bytes)."""
        assert batch % world == 0 and pool.layout == "hnd" and collective in ("rs_ag", "oneshot")
        self.collective = collective
        self._C = load()
        self.cfg, self.w, self.pool, self.rank, self.world = cfg, weights, pool, rank, world
        dev = pool.data.device
        self.device = dev
        self.max_batch = self.batch = batch
        self.rows = batch // world
        self.max_ctx = max_ctx
        H, D, L = cfg.hidden, cfg.head_dim, cfg.layers
        self.qh, self.kh = cfg.q_heads // world, cfg.kv_heads // world
        B = batch
        oneshot = collective == "oneshot"
        heap_bytes = 4 * B * H * 2 + world * B * 8 + 8192 + 4096 + (2 * world * B * H * 2 + 4096 if oneshot else 0)
        self.heap = SymmetricHeap(heap_bytes, rank, world, dev, group)
        hp = self.heap
        for name in ("agA", "agB", "rs0", "rs1"):
            hp.alloc(name, B * H * 2)
        if oneshot:
            for name in ("ar0", "ar1"):                  # [world][B][H] partials of the O and the down projection
                hp.alloc(name, world * B * H * 2)
        hp.alloc("am_slots", world * B * 8)
        hp.alloc("counters", 4096)
        # counter words: agA[world] | agB[world] | rs0 | rs1 | am[world]
        self.c_agA, self.c_agB, self.c_rs0, self.c_rs1, self.c_am = 0, 4 * world, 8 * world, 8 * world + 4, 8 * world + 8
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.resid = torch.zeros((B if oneshot else self.rows, H), **bf)      # replicated in the one-shot form
        self.xA = hp.local_tensor("agA", (B, H), torch.bfloat16)
        self.xB = hp.local_tensor("agB", (B, H), torch.bfloat16)
        self.qkv = torch.empty((B, (self.qh + 2 * self.kh) * D), **bf)
        self.q = torch.empty((B, self.qh, D), **bf)
        self.attn_out = torch.empty((B, self.qh, D), **bf)
        self.act = torch.empty((B, cfg.ffn // world), **bf)
        self.logits = torch.empty((B, weights.lm_head.shape[0]), **bf)
        self.next_ids = torch.zeros((B,), dtype=torch.int32, device=dev)
        self.ids = torch.zeros((B,), dtype=torch.int32, device=dev)
        self.positions = torch.zeros((B,), dtype=torch.int32, device=dev)
        self.ctx_lens = torch.ones((B,), dtype=torch.int32, device=dev)
        self.max_blocks = (max_ctx + 15) // 16
        self.block_table = torch.zeros((B, self.max_blocks), dtype=torch.int32, device=dev)
        self.inv_freq = ops.rope_inv_freq(cfg.rope_theta, dev, D)
        self.attn = ops.PagedAttention(dev, B, self.qh, self.kh, max_ctx, attn_chunk, impl=attn_impl)
        self.step_ctr = torch.zeros(1, dtype=torch.int32, device=dev)
        self.status = new_status(dev)
        self.ws = GemmWorkspace(dev)
        self.ws.status = self.status
        self.dummy = torch.empty((1, 1), **bf)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.graph_batch = batch
        self.kernels_per_step = 1 + 8 * L + 4        # embedding, 8 per layer, final norm, lm_head, argmax, step counter
        self.tiles_h = (H + 127) // 128
        if world > 1:
            dist.barrier(group)                      # every heap is mapped and zeroed before anyone pushes

    # ---- helpers ----
    def _ag(self, which: str, uses: int, use: int) -> tuple:
        off = self.c_agA if which == "A" else self.c_agB
        return (self.world, self.heap.ptr("counters", self.rank, off), self.step_ctr.data_ptr(), uses, use, self.rows, TIMEOUT_NS)

    def _rs(self, which: int) -> tuple:
        name, off = ("rs0", self.c_rs0) if which == 0 else ("rs1", self.c_rs1)
        return (self.world, self.rank, self.rows, self.heap.all_ptrs(name), self.heap.all_ptrs("counters", off))

    def _norm(self, rs_which: Optional[int], rs_use: int, w: torch.Tensor, ag_which: str) -> None:
        L = self.cfg.layers
        if rs_which is None:
            rs_buf, rs_ctr, seq = 0, 0, ()
        else:
            name, off = ("rs0", self.c_rs0) if rs_which == 0 else ("rs1", self.c_rs1)
            rs_buf, rs_ctr = self.heap.ptr(name, self.rank), self.heap.ptr("counters", self.rank, off)
            k_in = (self.cfg.q_heads // self.world) * self.cfg.head_dim if rs_which == 0 else self.cfg.ffn // self.world
            seq = (self.step_ctr.data_ptr(), L, rs_use, self._rs_arrivals(k_in))
        ag_name, ag_off = ("agA", self.c_agA) if ag_which == "A" else ("agB", self.c_agB)
        self._C.tp_norm(rs_buf, rs_ctr, seq, self.resid, w, self.heap.all_ptrs(ag_name),
                        self.heap.all_ptrs("counters", ag_off + 4 * self.rank), self.rank, self.cfg.eps, TIMEOUT_NS, self.status)

    def _config(self, M: int, N: int, K: int, gated: bool = False) -> Tuple[int, int, bool]:
        """(token tile, splits, cluster) of a GEMM of this engine; the arrival counts of the collectives are derived from the
        same choice."""
        if self.collective == "rs_ag":
            return (*pick_config(M, N, K, 148, gated, model=FUSED_TP), False)
        return choose_config(M, N, K, 148, gated)

    def _gemm(self, x, w, y, gated=False, ag=(), rs=()):
        M, K = x.shape
        N = w.shape[0] // 2 if gated else w.shape[0]
        ntok, splits, cluster = self._config(M, N, K, gated)
        if splits > 1 and cluster:
            self._C.gemm_tp(x, w, y, splits, gated, None, None, self.status, ag, rs, ntok, True)
        elif splits > 1:
            self.ws.ensure(self._C.gemm_workspace_floats(M, N, splits, gated, ntok), self._C.gemm_counter_count(M, N, gated, ntok))
            self._C.gemm_tp(x, w, y, splits, gated, self.ws.ws, self.ws.counters, self.status, ag, rs, ntok)
        else:
            self._C.gemm_tp(x, w, y, 1, gated, None, None, self.status, ag, rs, ntok)

    def _rs_arrivals(self, K: int) -> int:
        """Arrivals one reduce-scatter adds to a rank's counter: every output tile of every rank's GEMM."""
        ntok = self._config(self.batch, self.cfg.hidden, K)[0]
        return self.world * self.tiles_h * ((self.batch + ntok - 1) // ntok)

    def set_batch(self, ids: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor) -> None:
        b = ids.numel()
        self.ids[:b].copy_(ids)
        self.positions[:b].copy_(positions)
        self.ctx_lens[:b].copy_(positions + 1)
        self.block_table[:b, :block_table.shape[1]].copy_(block_table)

    # ---- one-shot all-reduce form ----
    def _ar(self, which: int) -> tuple:
        """Push descriptor of a GEMM whose partial tile goes to every rank's `ar<which>` buffer, slot [this rank][row]."""
        name = "ar0" if which == 0 else "ar1"
        off = self.c_rs0 if which == 0 else self.c_rs1
        return (self.world, self.rank, self.batch, self.heap.all_ptrs(name), self.heap.all_ptrs("counters", off), True)

    def _norm_ar(self, ar_which: Optional[int], use: int, w: torch.Tensor, x_out: torch.Tensor) -> None:
        """Sum of `world` partials + residual (replicated, updated in place) -> RMSNorm -> x_out, all local."""
        L = self.cfg.layers
        if ar_which is None:
            buf, ctr, seq = 0, 0, ()
        else:
            name, off = ("ar0", self.c_rs0) if ar_which == 0 else ("ar1", self.c_rs1)
            buf, ctr = self.heap.ptr(name, self.rank), self.heap.ptr("counters", self.rank, off)
            k_in = (self.cfg.q_heads // self.world) * self.cfg.head_dim if ar_which == 0 else self.cfg.ffn // self.world
            seq = (self.step_ctr.data_ptr(), L, use, self._rs_arrivals(k_in))
        self._C.tp_norm(buf, ctr, seq, self.resid, w, [x_out.data_ptr()], [0], self.rank, self.cfg.eps, TIMEOUT_NS, self.status,
                        rs_world=self.world)

    def _step_oneshot(self, b: int, max_ctx: int) -> None:
        cfg, w, L = self.cfg, self.w, self.cfg.layers
        ops.embedding(self.ids, w.embed, out=self.resid)                      # every rank embeds the whole batch
        for li, lw in enumerate(w.layers):
            self._norm_ar(None if li == 0 else 1, li - 1, lw.ln1, self.xA)
            self._gemm(self.xA, lw.qkv, self.qkv)
            ops.rope_append(self.qkv, lw.q_norm, lw.k_norm, self.pool, li, self.inv_freq, self.block_table, self.positions, self.qh,
                            cfg.eps, q_out=self.q)
            self.attn(self.q, self.pool, li, self.block_table, self.ctx_lens, max_ctx=max_ctx, out=self.attn_out)
            self._gemm(self.attn_out.view(b, -1), lw.o, self.dummy, rs=self._ar(0))
            self._norm_ar(0, li, lw.ln2, self.xB)
            self._gemm(self.xB, lw.gate_up, self.act, gated=True)
            self._gemm(self.act, lw.down, self.dummy, rs=self._ar(1))
        self._norm_ar(1, L - 1, w.final_norm, self.xA)
        self._gemm(self.xA, w.lm_head, self.logits)
        self._C.tp_argmax(self.logits, w.vocab_lo, self.rank, self.heap.all_ptrs("am_slots"),
                          self.heap.all_ptrs("counters", self.c_am + 4 * self.rank), self.heap.ptr("am_slots", self.rank),
                          self.heap.ptr("counters", self.rank, self.c_am), (self.step_ctr.data_ptr(), 1, 0, b), self.next_ids,
                          TIMEOUT_NS, self.status)
        self._C.step_increment(self.step_ctr)

    def _step(self, b: int, max_ctx: int) -> None:
        assert b == self.batch, "a tensor-parallel step always runs the full batch"
        if self.collective == "oneshot":
            return self._step_oneshot(b, max_ctx)
        cfg, w, L = self.cfg, self.w, self.cfg.layers
        r0 = self.rank * self.rows
        ops.embedding(self.ids[r0:r0 + self.rows], w.embed, out=self.resid)
        for li, lw in enumerate(w.layers):
            self._norm(None if li == 0 else 1, li - 1, lw.ln1, "A")
            self._gemm(self.xA, lw.qkv, self.qkv, ag=self._ag("A", L + 1, li))
            ops.rope_append(self.qkv, lw.q_norm, lw.k_norm, self.pool, li, self.inv_freq, self.block_table, self.positions, self.qh,
                            cfg.eps, q_out=self.q)
            self.attn(self.q, self.pool, li, self.block_table, self.ctx_lens, max_ctx=max_ctx, out=self.attn_out)
            self._gemm(self.attn_out.view(b, -1), lw.o, self.dummy, rs=self._rs(0))
            self._norm(0, li, lw.ln2, "B")
            self._gemm(self.xB, lw.gate_up, self.act, gated=True, ag=self._ag("B", L, li))
            self._gemm(self.act, lw.down, self.dummy, rs=self._rs(1))
        self._norm(1, L - 1, w.final_norm, "A")
        self._gemm(self.xA, w.lm_head, self.logits, ag=self._ag("A", L + 1, L))
        self._C.tp_argmax(self.logits, w.vocab_lo, self.rank, self.heap.all_ptrs("am_slots"),
                          self.heap.all_ptrs("counters", self.c_am + 4 * self.rank), self.heap.ptr("am_slots", self.rank),
                          self.heap.ptr("counters", self.rank, self.c_am), (self.step_ctr.data_ptr(), 1, 0, b), self.next_ids,
                          TIMEOUT_NS, self.status)
        self._C.step_increment(self.step_ctr)

    def profile_step(self, max_ctx: int) -> dict:
        """One eager step with a CUDA event after every kernel; returns milliseconds per kernel kind. Eager launches add
        host gaps, so read it for shares and for time spent waiting on peers, not for absolutes."""
        marks = []
        C = self._C
        orig = {n: getattr(C, n) for n in ("tp_norm", "gemm_tp", "tp_argmax", "step_increment", "rope_append", "paged_attn_decode", "embedding")}

        def wrap(name, fn):
            def f(*a, **k):
                r = fn(*a, **k)
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append((name, e))
                return r
            return f

        class Proxy:
            pass

        proxy = Proxy()
        for n in dir(C):
            if not n.startswith("__"):
                setattr(proxy, n, wrap(n, orig[n]) if n in orig else getattr(C, n))
        import skygdr_b200.ops.small as small
        import skygdr_b200.ops.attention as att

        saved = (self._C, small.load, self.attn._C)
        self._C = proxy
        small.load = lambda: proxy
        self.attn._C = proxy
        try:
            start = torch.cuda.Event(enable_timing=True)
            start.record()
            self._step(self.batch, max_ctx)
            torch.cuda.synchronize(self.device)
        finally:
            self._C, small.load, self.attn._C = saved
        out, prev = {}, start
        for name, e in marks:
            out[name] = out.get(name, 0.0) + prev.elapsed_time(e)
            prev = e
        out["total"] = start.elapsed_time(marks[-1][1])
        return out

    _advance = Qwen3Decoder._advance
    capture = Qwen3Decoder.capture

    # A step's kernels wait (bounded) for every peer, so a step launched after a peer has gone only burns its time-outs.
    # With a ``liveness.RankWatch`` attached, the host checks the peers before every launch and raises ``PeerLost`` instead.
    watch = None

    def attach_watch(self, watch) -> None:
        self.watch = watch

    def step(self, *args, **kwargs) -> torch.Tensor:
        if self.watch is not None:
            self.watch.guard()
        return Qwen3Decoder.step(self, *args, **kwargs)

    def replay(self) -> torch.Tensor:
        if self.watch is not None:
            self.watch.guard()
        return Qwen3Decoder.replay(self)

    def check_status(self) -> str:
        """"OK", or the first non-OK status a kernel of this engine left behind: the GEMM, norm and argmax kernels share one
        status word, the attention kernels have their own."""
        torch.cuda.synchronize(self.device)
        for st in (read_status(self.status), read_status(self.attn.status)):
            if st["status"] != 0:
                return f"{st['status_name']}:{st['detail']}"
        return "OK"

    def clear_status(self) -> None:
        """Back to "OK" after a wait that gave up. Kernels skip their peer waits while the status is not OK (one lost peer must
        not cost a timeout per kernel), so a job that carries on after such an event clears it on every rank between two steps.
        Arrival counters keep counting through a skipped wait, so the ranks stay in step."""
        torch.cuda.synchronize(self.device)
        self.status.zero_()
        self.attn.status.zero_()

    def bytes_per_step(self, ctx: torch.Tensor) -> int:
        return _bytes_per_step(self.cfg, self.w, ctx, self.kh, self.batch)


def _bytes_per_step(cfg: Qwen3Config, w: Qwen3Weights, ctx: torch.Tensor, kv_heads_local: int, batch: int) -> int:
    weights = w.nbytes() - w.embed.numel() * 2 + batch * cfg.hidden * 2
    kv = int(ctx.sum()) * cfg.layers * 2 * kv_heads_local * cfg.head_dim * 2
    return weights + kv


def build_decode_engine(cfg: Qwen3Config, device: torch.device, rank: int, world: int, ctx: torch.Tensor, extra_tokens: int,
                        seed: int = 0, kv_init: str = "normal", attn_chunk: int = 0, attn_impl: str = "tc",
                        collective: str = "oneshot"):
    """Weights shard, KV pool sized for ``ctx`` (+ ``extra_tokens`` of growth per sequence), randomly permuted block
    table, and the decode engine for this rank. Every rank passes the same ``ctx`` and ``seed``. ``attn_chunk`` 0: the tokens
    per attention CTA are planned from the context lengths (``ops.attention.plan_chunk_tokens``)."""
    batch = ctx.numel()
    if not attn_chunk:
        from ..ops.attention import plan_chunk_tokens

        sms = torch.cuda.get_device_properties(device).multi_processor_count if torch.cuda.is_available() else 148
        # Measured on B200 with the benchmark's batch: the planned size against 1024 tokens gave +2.4 % of the decode step at 8 KV heads
        # per GPU and +1.1 % at 4, but -0.5 % at 2 (64 sequences per rank: the model overrates what is to be won there), so ranks
        # with fewer than 4 KV heads keep 1024.
        plan = attn_impl == "tc" and cfg.kv_heads // world >= 4
        attn_chunk = plan_chunk_tokens([int(c) + extra_tokens // 2 for c in ctx], cfg.kv_heads // world, sms) if plan else 1024
    weights = Qwen3Weights(cfg, device, seed=seed, tp_rank=rank, tp_world=world)
    geom = KVGeometry(cfg.layers, cfg.kv_heads // world, cfg.head_dim)
    blocks_per_seq = [(int(c) + extra_tokens + 15) // 16 for c in ctx]
    nblocks = sum(blocks_per_seq) + 1
    pool = PagedKVPool(geom, nblocks, "hnd", device=device)
    if kv_init == "normal":
        # filled in slices to keep the temporary small
        step = max(1, (1 << 28) // (geom.block_elems))
        for i in range(0, nblocks, step):
            pool.data[i:i + step].normal_()
    max_ctx = int(ctx.max()) + extra_tokens + 1
    max_blocks = (max_ctx + 15) // 16
    g = torch.Generator().manual_seed(seed + 12345)
    perm = (torch.randperm(nblocks - 1, generator=g) + 1).int()      # block 0 stays a scratch block for padded table entries
    table = torch.zeros((batch, max_blocks), dtype=torch.int32)
    o = 0
    for i, nb in enumerate(blocks_per_seq):
        table[i, :nb] = perm[o:o + nb]
        o += nb
    if world == 1:
        eng = Qwen3Decoder(cfg, weights, pool, batch, max_ctx, attn_chunk, attn_impl)
    else:
        eng = TPDecoder(cfg, weights, pool, batch, max_ctx, rank, world, attn_chunk, attn_impl=attn_impl, collective=collective)
    return eng, table
