"""Continuous batching (skygdr_b200/models/serving.py) against a stand-in engine on the CPU.

The stand-in keeps its "KV cache" in blocks addressed through the block table exactly as the real engine does (token at
position p lives in block table[p // 16], offset p % 16) and its next token is a function of the whole history read back
through the table, so a wrong table row, a block shared by two sequences or a stale position changes the output."""
import random

import pytest
import torch

from skygdr_b200 import ops
from skygdr_b200.models import ContinuousBatcher, Request

VOCAB = 997


def next_token(history):
    return (sum((i + 1) * t for i, t in enumerate(history)) * 31 + len(history)) % VOCAB


class StandInEngine:
    def __init__(self, max_batch, num_blocks):
        self.max_batch, self.device = max_batch, torch.device("cpu")
        self.kv = torch.full((num_blocks, 16), -1, dtype=torch.int64)
        self.steps = 0

    def _history(self, row, n):
        return [int(self.kv[int(row[p // 16]), p % 16]) for p in range(n)]

    def prefill(self, ids, seq_lens, table):
        assert len(seq_lens) == 1 and table.shape[0] == 1
        for p, t in enumerate(ids.tolist()):
            self.kv[int(table[0, p // 16]), p % 16] = t
        logits = torch.zeros((1, VOCAB))
        logits[0, next_token(self._history(table[0], seq_lens[0]))] = 1.0
        return logits

    def set_batch(self, ids, positions, table):
        self.ids, self.pos, self.table = ids.clone(), positions.clone(), table.clone()

    def step(self):
        self.steps += 1
        out = torch.zeros(self.max_batch, dtype=torch.int32)
        for s in range(self.max_batch):
            p = int(self.pos[s])
            self.kv[int(self.table[s, p // 16]), p % 16] = int(self.ids[s])          # append, as RoPE + KV append does
            out[s] = next_token(self._history(self.table[s], p + 1))
        return out


def expected(prompt, max_new, eos):
    hist, out = list(prompt), []
    while len(out) < max_new:
        t = next_token(hist)
        out.append(t)
        hist.append(t)
        if eos is not None and t == eos:
            break
    return out


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_every_request_gets_the_tokens_it_would_get_alone(seed):
    rng = random.Random(seed)
    num_blocks, slots = 40, 4
    eng = StandInEngine(slots, num_blocks)
    alloc = ops.BlockAllocator(num_blocks, max_seqs=slots, max_ctx=256)
    b = ContinuousBatcher(eng, alloc)
    reqs, want = [], {}
    for rid in range(25):
        prompt = [rng.randrange(VOCAB) for _ in range(rng.choice([1, 3, 15, 16, 17, 40, 90]))]
        max_new = rng.choice([1, 2, 5, 20, 60])
        eos = rng.choice([None, None, rng.randrange(VOCAB)])
        reqs.append(Request(rid, torch.tensor(prompt), max_new, eos))
        want[rid] = expected(prompt, max_new, eos)
    got = {}
    pending = list(reqs)
    while pending or not b.idle():
        for _ in range(rng.randrange(0, 3)):                 # requests arrive while the batch is running
            if pending:
                b.submit(pending.pop(0))
        for rid, tok in b.step():
            got.setdefault(rid, []).append(tok)
        owned = [x for k in range(slots) for x in alloc.blocks_of(k).tolist()]
        assert len(owned) == len(set(owned)) and 0 not in owned
        assert b.running <= slots
    assert got == want
    assert all(r.finished and r.output == want[r.req_id] for r in reqs)
    assert alloc.free_blocks == alloc.capacity                # everything was given back
    assert eng.steps == b.steps and b.steps < sum(len(v) for v in want.values())     # sequences really shared steps


def test_admission_waits_for_memory_and_refuses_what_can_never_fit():
    eng = StandInEngine(2, 8)
    alloc = ops.BlockAllocator(8, max_seqs=2, max_ctx=128)    # 7 usable blocks = 112 tokens
    b = ContinuousBatcher(eng, alloc)
    with pytest.raises(MemoryError):
        b.submit(Request(0, torch.tensor([1] * 100), 20))     # 120 tokens: more than the pool will ever have
    b.submit(Request(1, torch.tensor([1] * 60), 4))           # 4 blocks
    b.submit(Request(2, torch.tensor([2] * 60), 4))           # 4 more: has to wait although a slot is free
    b.submit(Request(3, torch.tensor([3] * 2), 2))            # small, but first come first served: it does not overtake
    first = b.step()                                          # admits request 1 (its first token comes from the prefill), steps once
    assert b.running == 1 and len(b.waiting) == 2 and [r for r, _ in first] == [1, 1]
    out = b.run_until_idle()
    out[1] = [t for _, t in first] + out[1]
    assert set(out) == {1, 2, 3} and [len(out[k]) for k in (1, 2, 3)] == [4, 4, 2]
    assert out[2] == expected([2] * 60, 4, None)


def test_batcher_drives_the_real_engine_class_with_stubbed_kernels(monkeypatch):
    """The batcher against Qwen3Decoder itself (kernels replaced by recorders that return zeros): signatures, devices and
    shapes fit, every request gets its number of tokens, and idle slots keep running on block 0."""
    from test_ops_cpu import _stub_kernels

    from skygdr_b200.models import Qwen3Config, Qwen3Decoder, Qwen3Weights

    calls = []
    _stub_kernels(monkeypatch, calls)
    cfg = Qwen3Config.tiny(layers=2)
    pool = ops.PagedKVPool(cfg.geometry, 32, "hnd", device="cpu")
    eng = Qwen3Decoder(cfg, Qwen3Weights(cfg, "cpu", seed=0), pool, max_batch=3, max_ctx=128, attn_chunk=128)
    b = ContinuousBatcher(eng, ops.BlockAllocator(32, max_seqs=3, max_ctx=128), use_graph=False)
    for rid, (n, new) in enumerate([(20, 3), (5, 6), (33, 2), (9, 4)]):
        b.submit(Request(rid, torch.randint(0, cfg.vocab, (n,)), new))
    out = b.run_until_idle(max_steps=50)
    assert {k: len(v) for k, v in out.items()} == {0: 3, 1: 6, 2: 2, 3: 4}
    assert b.alloc.free_blocks == b.alloc.capacity and b.idle()
    assert sum(1 for c in calls if c[0] == "prefill_attn") == 4 * cfg.layers   # one prefill per request
