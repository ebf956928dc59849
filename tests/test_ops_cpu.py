"""Host-side helpers of the ops layer, on CPU tensors: pool geometry, reference gathers, fp8 packing oracle, the GEMM
shape chooser (with a stubbed extension), the attention oracle."""
import math
import types

import pytest
import torch


def test_geometry_and_pool_views():
    from skygdr_b200.ops.kv_cache import KVGeometry, PagedKVPool

    g = KVGeometry()
    assert g.bytes_per_token() == 147456 and g.page_elems == 16 * 8 * 128 and g.block_elems == 36 * 2 * g.page_elems
    assert g.blocks_for(1) == 1 and g.blocks_for(16) == 1 and g.blocks_for(17) == 2
    small = KVGeometry(layers=2, kv_heads=2)
    nhd = PagedKVPool(small, 5, "nhd", device="cpu", dtype=torch.float32)
    hnd = PagedKVPool(small, 5, "hnd", device="cpu", dtype=torch.float32)
    assert nhd.data.shape == (5, 2, 2, 16, 2, 128) and hnd.data.shape == (5, 2, 2, 2, 16, 128)
    assert nhd.strides == (small.block_elems, 2 * small.page_elems, small.page_elems) and hnd.head_stride == 16 * 128
    nhd.data.normal_()
    hnd.data.copy_(nhd.data.permute(0, 1, 2, 4, 3, 5))
    blocks = torch.tensor([3, 0, 4])
    assert torch.equal(nhd.gather_reference(blocks), hnd.gather_reference(blocks))


def test_reference_transfer_and_link_bytes():
    from skygdr_b200.ops.kv_cache import KVGeometry, PagedKVPool
    from skygdr_b200.ops.kv_transfer import link_bytes, reference_transfer

    g = KVGeometry(layers=1, kv_heads=4)
    src = PagedKVPool(g, 3, "nhd", device="cpu", dtype=torch.float32)
    src.data.copy_(torch.arange(src.data.numel(), dtype=torch.float32).view_as(src.data))
    out = reference_transfer(src, torch.tensor([2, 0]), slice(1, 3))
    assert out.shape == (2, 1, 2, 2, 16, 128)
    assert torch.equal(out[0, 0, 1, 0, 5], src.data[2, 0, 1, 5, 1])          # head 1 of the slice = source head 1
    assert link_bytes(g, 10) == 10 * g.block_elems * 2
    assert link_bytes(g, 10, n_dst=3, replicate=True) == 3 * link_bytes(g, 10)
    assert link_bytes(g, 10, fp8=True) == 10 * (g.block_elems + g.block_elems // 32)


def test_fp8_mx_oracle_properties():
    from skygdr_b200.ops.kv_transfer import fp8_mx_reference

    torch.manual_seed(0)
    x = torch.randn(4, 64) * torch.tensor([1e-3, 1.0, 50.0, 1e4])[:, None]
    x[0, :32] = 0
    q, s = fp8_mx_reference(x.bfloat16())
    assert q.shape == (4, 64) and s.shape == (4, 2) and q.dtype == torch.uint8
    back = q.view(torch.float8_e4m3fn).float() * torch.exp2(s.float() - 127).repeat_interleave(32, -1)
    assert int(s[0, 0]) == 0 and float(back[0, :32].abs().max()) == 0.0        # all-zero group: smallest scale, zeros
    rel = (back - x.bfloat16().float()).abs().max(-1).values / x.abs().max(-1).values
    assert float(rel.max()) < 0.07                                              # e4m3 keeps 3 mantissa bits
    scaled = x.bfloat16().float().view(4, 2, 32) * torch.exp2(127 - s.float())[..., None]
    assert float(scaled.abs().max()) <= 448.0                                   # nothing saturates under the chosen scale
    assert float(scaled.view(4, 2, 32)[1:].abs().amax(-1).min()) > 224.0        # ... and the scale is the smallest such power of two


def test_pick_config_rules(monkeypatch):
    import importlib

    g = importlib.import_module("skygdr_b200.ops.gemm")           # the package re-exports a function of the same name

    monkeypatch.setattr(g, "load", lambda: types.SimpleNamespace(
        gemm_pick_ntok=lambda M, gated: 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128))
    for M, N, K, gated in [(16, 6144, 4096, False), (16, 12288, 4096, True), (128, 768, 4096, False), (128, 4096, 512, False),
                           (16, 151936, 4096, False), (1, 128, 64, False), (300, 1024, 2048, False)]:
        ntok, s = g.pick_config(M, N, K, 148, gated)
        assert ntok in (16, 32, 64, 128, 256) and 1 <= s <= 16
        assert s == 1 or (K // 64) // s >= 4                                    # a split keeps at least 4 k-blocks
        assert not (gated and ntok > 128)
    assert g.pick_config(16, 151936, 4096, 148)[1] == 1                          # many tiles: never split
    assert g.pick_config(128, 768, 4096, 148)[1] > 1                             # six tiles: must split
    assert g.pick_config(16, 6144, 4096, 148, fixed_ntok=16)[0] == 16
    # the fused tensor-parallel GEMMs keep the tile/split choices under which the TP step was tuned end to end
    tuned = {(128, 768, 4096, False): (32, 5), (128, 4096, 512, False): (32, 1), (128, 1536, 4096, True): (64, 5), (128, 4096, 1536, False): (64, 2),
             (32, 3072, 4096, False): (32, 5), (32, 4096, 2048, False): (32, 4), (32, 6144, 4096, True): (32, 3), (32, 4096, 6144, False): (32, 4)}
    for (M, N, K, gated), want in tuned.items():
        assert g.pick_config(M, N, K, 148, gated, model=g.FUSED_TP) == want
    assert g.pick_config(128, 768, 4096, 148)[0] == 16                           # alone, small token tiles win


def test_attention_oracle_matches_dense_softmax():
    from skygdr_b200.ops.attention import paged_attn_reference
    from skygdr_b200.ops.kv_cache import KVGeometry, PagedKVPool

    torch.manual_seed(1)
    g = KVGeometry(layers=1, kv_heads=2)
    pool = PagedKVPool(g, 6, "hnd", device="cpu", dtype=torch.float32)
    pool.data.normal_()
    table = torch.tensor([[4, 1, 0], [2, 5, 3]], dtype=torch.int32)
    ctx = torch.tensor([20, 48], dtype=torch.int32)
    q = torch.randn(2, 4, 128)
    out = paged_attn_reference(q, pool, 0, table, ctx)
    b, h = 0, 3
    k = torch.cat([pool.data[4, 0, 0, 1], pool.data[1, 0, 0, 1]])[:20]          # query head 3 reads kv head 1
    v = torch.cat([pool.data[4, 0, 1, 1], pool.data[1, 0, 1, 1]])[:20]
    p = torch.softmax(q[b, h] @ k.t() / math.sqrt(128), -1)
    assert torch.allclose(out[b, h], p @ v, atol=1e-5)


@pytest.mark.parametrize("layout", ["hnd", "nhd"])
def test_prefill_oracle_matches_torch_sdpa(layout):
    """The oracle of the prefill attention kernel (gather pages, causal softmax in fp32) against torch's own attention."""
    from skygdr_b200.ops.attention import prefill_attn_reference
    from skygdr_b200.ops.kv_cache import KVGeometry, PagedKVPool

    torch.manual_seed(2)
    g = KVGeometry(layers=2, kv_heads=2)
    lens = [5, 33, 16]
    pool = PagedKVPool(g, 12, layout, device="cpu", dtype=torch.float32)
    pool.data.normal_()
    table = torch.tensor([[3, 0, 0], [7, 1, 9], [4, 0, 0]], dtype=torch.int32)
    q = torch.randn(sum(lens), 4, 128)
    out = prefill_attn_reference(q, pool, 1, table, lens)
    o = 0
    for s, n in enumerate(lens):
        nb = (n + 15) // 16
        kv = pool.data[table[s, :nb].long(), 1]
        if layout == "nhd":
            kv = kv.permute(0, 1, 3, 2, 4)
        k = kv[:, 0].permute(1, 0, 2, 3).reshape(2, nb * 16, 128)[:, :n]
        v = kv[:, 1].permute(1, 0, 2, 3).reshape(2, nb * 16, 128)[:, :n]
        want = torch.nn.functional.scaled_dot_product_attention(q[o:o + n].transpose(0, 1)[None], k[None], v[None], is_causal=True, enable_gqa=True)
        assert torch.allclose(out[o:o + n], want[0].transpose(0, 1), atol=1e-5)
        o += n


def test_library_send_recv_handoff_moves_paged_kv_between_two_ranks(tmp_path):
    """The comparison arm for the transfer kernel (gather + layout change, library send / recv, scatter) as two gloo
    ranks: the receiver must end up with head-major copies of exactly the sender's blocks, in its own block order."""
    import json
    import os
    import socket
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "lib.json"
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), os.path.join(root, "benchmarks", "config2_library_sendrecv.py"), "--device", "cpu",
                        "--requests", "2", "--min-tokens", "64", "--max-tokens", "1024", "--layers", "2", "--blocks-per-message", "7",
                        "--out", str(out)], capture_output=True, text=True, timeout=300, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.load(open(out))
    assert d["arms"]["send_recv_paged"]["exact"] is True
    assert d["arms"]["send_recv_paged"]["gb"] == d["arms"]["send_recv_contiguous"]["gb"] > 0       # same payload in both arms
    assert d["config"]["backend"] == "gloo"


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_shards_reproduce_the_unsharded_forward_on_cpu_ranks(world):
    """Shard layout of the weights (heads, FFN columns, O / down input slices, vocabulary ranges) checked by gloo ranks:
    the plain-PyTorch tensor-parallel forward on the shards must give the unsharded logits."""
    import json
    import os
    import socket
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
                        "--master-port", str(port), os.path.join(root, "tests", "multi", "tp_oracle_worker.py")],
                       capture_output=True, text=True, timeout=300, cwd=root)
    assert r.returncode == 0, r.stderr[-3000:]
    d = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert d["world"] == world and d["covered"] and d["argmax_agrees"] and d["clear_rows"] > 0
    assert d["rel_err_max"] < 0.03, d             # bf16 rounding of per-rank partial sums is the only difference


def _simulate_persistent_gemm_pipeline(n_my_tiles, nkb, stages, seed):
    """The barrier protocol of gemm_persistent_kernel (skygdr_b200/csrc/kernels/gemm_tcgen05.cu) as three coroutines under a
    random scheduler: TMA producer, MMA issuer, epilogue. mbarriers are modelled as phase counters: a wait on parity P
    passes once the barrier's current phase has parity != P. Asynchronous completions (TMA bytes landing, tcgen05.commit
    arrivals) are events that the scheduler delivers at random later times. Returns the order in which the epilogue saw
    (tile, checksum) and raises on any hazard: a ring slot overwritten before its MMAs read it, an accumulator overwritten
    before it was drained, an MMA on a slot whose data has not landed."""
    import random

    rng = random.Random(seed)
    phase = {("full", s): 0 for s in range(stages)} | {("empty", s): 0 for s in range(stages)} | \
            {("acc_full", b): 0 for b in range(2)} | {("acc_empty", b): 0 for b in range(2)}
    slot = [None] * stages            # (tile, kb) whose data is in the slot, or None while free / in flight
    slot_busy = [False] * stages      # loaded and not yet read by the tensor core
    acc = [None, None]                # per accumulator: [tile, number of k-blocks accumulated, drained?]
    pending = []                      # asynchronous completions not yet delivered: callables
    seen = []

    def passed(bar, parity):
        return (phase[bar] & 1) != parity

    def producer():
        it = 0
        for j in range(n_my_tiles):
            for kb in range(nkb):
                s = it % stages
                if it >= stages:
                    while not passed(("empty", s), ((it // stages) - 1) & 1):
                        yield
                assert not slot_busy[s], ("slot overwritten before it was read", j, kb)
                slot[s] = None

                def land(s=s, j=j, kb=kb):
                    slot[s] = (j, kb)
                    slot_busy[s] = True
                    phase[("full", s)] += 1
                pending.append(land)
                it += 1
                yield

    def mma():
        it = 0
        for j in range(n_my_tiles):
            buf = j & 1
            if j >= 2:
                while not passed(("acc_empty", buf), ((j >> 1) - 1) & 1):
                    yield
            assert acc[buf] is None or acc[buf][2], ("accumulator overwritten before it was drained", j)
            acc[buf] = [j, 0, False]
            for kb in range(nkb):
                s = it % stages
                while not passed(("full", s), (it // stages) & 1):
                    yield
                assert slot[s] == (j, kb), ("MMA on a slot that does not hold its operands", j, kb, slot[s])
                acc[buf][1] += 1

                def read_done(s=s):                 # tcgen05.commit -> empty barrier, once the MMAs have read the slot
                    slot_busy[s] = False
                    phase[("empty", s)] += 1
                pending.append(read_done)
                it += 1
                yield
            pending.append(lambda buf=buf: phase.__setitem__(("acc_full", buf), phase[("acc_full", buf)] + 1))
            yield

    def epilogue():
        for j in range(n_my_tiles):
            buf = j & 1
            while not passed(("acc_full", buf), (j >> 1) & 1):
                yield
            assert acc[buf][0] == j and acc[buf][1] == nkb, ("epilogue read an incomplete or foreign accumulator", j, acc[buf])
            seen.append(j)
            yield                                    # the loads and stores of the tile take a while
            acc[buf][2] = True
            phase[("acc_empty", buf)] += 1           # plain arrive: immediate

    live = [producer(), mma(), epilogue()]
    steps = 0
    while live:
        steps += 1
        assert steps < 200000, "the pipeline stopped making progress"
        # asynchronous completions are delivered in issue order per kind, at random times
        if pending and (rng.random() < 0.5 or len(live) == 0):
            pending.pop(0)()
            continue
        g = rng.choice(live)
        try:
            next(g)
        except StopIteration:
            live.remove(g)
        if not live:
            while pending:
                pending.pop(0)()
    return seen


@pytest.mark.parametrize("n_my_tiles,nkb,stages", [(1, 1, 4), (1, 9, 4), (2, 3, 4), (3, 64, 4), (7, 5, 6), (5, 1, 4), (4, 2, 8), (9, 16, 4)])
def test_persistent_gemm_pipeline_protocol(n_my_tiles, nkb, stages):
    """Parities and ordering of the four barrier families of the persistent GEMM, for few and many tiles per CTA, k-loops shorter
    and longer than the ring: under many random interleavings every tile reaches the epilogue complete and in order."""
    for seed in range(40):
        assert _simulate_persistent_gemm_pipeline(n_my_tiles, nkb, stages, seed) == list(range(n_my_tiles))


def _simulate_tp_collectives(collective, world, layers, steps, seed):
    """The cross-rank protocol of parallel.tp.TPDecoder as a model: every rank runs its kernels in stream order, a kernel
    runs only when the counters it waits for have reached the value it computes from (step, use), its remote writes land in
    the peers' buffers and its arrivals bump the peers' counters. Ranks advance under a random scheduler, so any rank can be
    arbitrarily late. Every buffer slot carries the tag of what was last written and whether its owner has read it:
    overwriting an unread slot, or reading a slot that holds something else than expected, is a hazard. Counters only grow.
    Returns the number of kernels run; raises on a hazard or when no rank can make progress."""
    import random

    rng = random.Random(seed)
    L, W = layers, world
    ctr = [dict() for _ in range(W)]                   # per rank: counter name -> value
    buf = [dict() for _ in range(W)]                   # per rank: (buffer, slot) -> [tag, read?]

    def get(r, name):
        return ctr[r].get(name, 0)

    def write(dst, name, slot, tag):
        cur = buf[dst].get((name, slot))
        assert cur is None or cur[1], ("overwrote unread data", name, "on rank", dst, "slot", slot, "old", cur, "new", tag)
        buf[dst][(name, slot)] = [tag, False]

    def read(r, name, slot, tag):
        cur = buf[r].get((name, slot))
        assert cur is not None and cur[0] == tag, ("read something else than expected", name, r, slot, cur, tag)
        cur[1] = True

    def program(r):
        """Yields (wait, action) pairs: wait is a list of (counter, value) that must hold on rank r before action() runs."""
        for step in range(steps):
            for li in range(L + 1):                    # li == L: the final norm and lm_head
                # ---- norm in front of QKV / lm_head: sums the previous layer's down-projection partials ----
                prev = ("down", step, li - 1)
                if collective == "oneshot":
                    waits = [("rs1", (step * L + li) * W)] if li > 0 else []

                    def k_norm1(li=li, prev=prev):
                        if li > 0:
                            for src in range(W):
                                read(r, "ar1", src, prev)
                    yield waits, k_norm1
                    yield [], (lambda: None)           # QKV or lm_head GEMM on local, replicated activations
                else:
                    waits = [("rs1", (step * L + li) * W)] if li > 0 else []

                    def k_norm1(step=step, li=li, prev=prev):
                        if li > 0:
                            for src in range(W):
                                read(r, "rs1", src, prev)
                        for d in range(W):             # all-gather push: this rank's rows into everybody's buffer A
                            write(d, "agA", r, ("A", step, li))
                            ctr[d][("agA", r)] = get(d, ("agA", r)) + 1
                    yield waits, k_norm1

                    def k_qkv(step=step, li=li):
                        for src in range(W):
                            read(r, "agA", src, ("A", step, li))
                    yield [(("agA", src), step * (L + 1) + li + 1) for src in range(W)], k_qkv
                if li == L:
                    break
                yield [], (lambda: None)               # RoPE + append, attention: local

                # ---- O projection: partials to the peers ----
                def k_o(step=step, li=li):
                    for d in range(W):
                        write(d, "ar0" if collective == "oneshot" else "rs0", r, ("o", step, li))
                        ctr[d]["rs0"] = get(d, "rs0") + 1
                yield [], k_o

                # ---- norm in front of gate/up ----
                def k_norm2(step=step, li=li):
                    for src in range(W):
                        read(r, "ar0" if collective == "oneshot" else "rs0", src, ("o", step, li))
                    if collective != "oneshot":
                        for d in range(W):
                            write(d, "agB", r, ("B", step, li))
                            ctr[d][("agB", r)] = get(d, ("agB", r)) + 1
                yield [("rs0", (step * L + li + 1) * W)], k_norm2
                if collective == "oneshot":
                    yield [], (lambda: None)           # gate/up on local activations
                else:
                    def k_gu(step=step, li=li):
                        for src in range(W):
                            read(r, "agB", src, ("B", step, li))
                    yield [(("agB", src), step * L + li + 1) for src in range(W)], k_gu

                # ---- down projection: partials to the peers ----
                def k_down(step=step, li=li):
                    for d in range(W):
                        write(d, "ar1" if collective == "oneshot" else "rs1", r, ("down", step, li))
                        ctr[d]["rs1"] = get(d, "rs1") + 1
                yield [], k_down
            # ---- vocabulary-parallel argmax: candidates to everybody, then wait for everybody's ----
            def k_am_push(step=step):
                for d in range(W):
                    write(d, "am", r, ("am", step))
                    ctr[d]["am"] = get(d, "am") + 1
            yield [], k_am_push

            def k_am_pick(step=step):
                for src in range(W):
                    read(r, "am", src, ("am", step))
            yield [("am", (step + 1) * W)], k_am_pick

    progs = [program(r) for r in range(W)]
    nxt = [next(p) for p in progs]
    done, ran = [False] * W, 0
    while not all(done):
        ready = [r for r in range(W) if not done[r] and all(get(r, c) >= v for c, v in nxt[r][0])]
        assert ready, ("no rank can make progress", [(r, nxt[r][0]) for r in range(W) if not done[r]])
        # a biased pick: now and then one rank races ahead as far as it can, or stalls for a long time
        r = rng.choice(ready) if rng.random() < 0.7 else ready[0]
        nxt[r][1]()
        ran += 1
        try:
            nxt[r] = next(progs[r])
        except StopIteration:
            done[r] = True
    return ran


@pytest.mark.parametrize("collective", ["rs_ag", "oneshot"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_counter_protocol_has_no_deadlock_and_no_overwrite(collective, world):
    """Both collective forms of the tensor-parallel step (reduce-scatter + all-gather with a token-sharded residual stream,
    and the one-shot all-reduce with replicated activations): counters computed from (step, use) are always reached, and no
    rank ever overwrites a peer's buffer before the peer has read it, however far ranks drift apart. Three steps, so the
    reuse of every buffer across steps is covered."""
    for seed in range(25):
        assert _simulate_tp_collectives(collective, world, layers=3, steps=3, seed=seed) > 0


def test_gumbel_max_reference_samples_the_softmax():
    """The sampling rule restated on the CPU (hash -> uniform -> Gumbel noise -> argmax): over many positions the picked tokens
    follow softmax(logits / T), the same (seed, position) always picks the same token, and a low temperature approaches greedy."""
    from skygdr_b200 import ops

    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5, -3.0]]).to(torch.bfloat16)
    T, n = 0.8, 40000
    rows = logits.repeat(n, 1)
    pos = torch.arange(n, dtype=torch.int32)
    ids, _ = ops.sample_reference(rows, T, seed=123, positions=pos)
    freq = torch.bincount(ids.long(), minlength=6).float() / n
    want = torch.softmax(logits[0].float() / T, -1)
    assert float((freq - want).abs().max()) < 0.01, (freq, want)
    again, _ = ops.sample_reference(rows[:100], T, seed=123, positions=pos[:100])
    assert torch.equal(again, ids[:100])
    other, _ = ops.sample_reference(rows[:2000], T, seed=124, positions=pos[:2000])
    assert float((other != ids[:2000]).float().mean()) > 0.3                     # another seed is another stream
    cold, _ = ops.sample_reference(rows[:2000], 0.02, seed=5, positions=pos[:2000])
    assert float((cold == 0).float().mean()) > 0.999
    from skygdr_b200.ops.small import sample_noise_reference

    u = sample_noise_reference(7, pos[:64], 64, 4096)
    assert 0.0 < float(u.min()) and float(u.max()) < 1.0 and abs(float(u.mean()) - 0.5) < 0.005


def test_checkpoint_loader_and_reference_forward_match_the_hugging_face_qwen3():
    """A tiny random Qwen3 built by the transformers library, loaded through Qwen3Weights.from_state_dict: this package's
    PyTorch forward (the oracle of all its GPU engines) must give the library's logits, which pins the architecture (QK-norm
    before RoPE, rotate-half RoPE, GQA head order, gated SiLU MLP, norm placement) and the fused / sharded weight layouts."""
    transformers = pytest.importorskip("transformers")
    from skygdr_b200.models import Qwen3Config, Qwen3Weights, reference_forward

    hc = transformers.Qwen3Config(vocab_size=300, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                                  num_key_value_heads=2, head_dim=128, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                                  max_position_embeddings=512)
    torch.manual_seed(0)
    hf = transformers.Qwen3ForCausalLM(hc).eval().to(torch.bfloat16)
    with torch.no_grad():                                            # make the norms' gains non-trivial
        for name, prm in hf.named_parameters():
            if "norm" in name:
                prm.copy_(1.0 + 0.2 * torch.randn_like(prm))
    cfg = Qwen3Config.from_hf(hc)
    assert (cfg.layers, cfg.hidden, cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab) == (2, 256, 4, 2, 128, 512, 300)
    sd = hf.state_dict()
    w = Qwen3Weights.from_state_dict(cfg, sd, device="cpu")
    ids = torch.randint(0, 300, (23,))
    with torch.no_grad():
        want = hf.float()(ids[None]).logits[0]
    got = reference_forward(cfg, w, ids)
    err = float((got - want).abs().max() / want.abs().max())
    assert err < 0.03, err                                           # bf16 rounding of activations between the layers is the only difference
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) > 0.85
    # the shards of a two-way split are the matching slices of the full tensors
    s1 = Qwen3Weights.from_state_dict(cfg, sd, device="cpu", tp_rank=1, tp_world=2)
    D = cfg.head_dim
    assert torch.equal(s1.layers[0].qkv[:2 * D], w.layers[0].qkv[2 * D:4 * D])                   # q heads 2-3
    assert torch.equal(s1.layers[0].qkv[2 * D:3 * D], w.layers[0].qkv[4 * D + D:4 * D + 2 * D])  # k head 1
    assert torch.equal(s1.layers[1].o, w.layers[1].o[:, 2 * D:]) and torch.equal(s1.layers[1].down, w.layers[1].down[:, 256:])
    assert torch.equal(s1.layers[1].gate_up[:256], w.layers[1].gate_up[256:512]) and torch.equal(s1.lm_head, w.lm_head[150:])


def test_block_allocator_never_hands_a_block_to_two_sequences():
    """Random admit / grow / finish traffic over a small pool: every live block belongs to exactly one slot, block 0 stays out
    of circulation, rows cover their contexts, a refused request leaves the row untouched, and everything comes back."""
    import random

    from skygdr_b200 import ops

    rng = random.Random(3)
    a = ops.BlockAllocator(num_blocks=64, max_seqs=6, max_ctx=400)
    assert a.capacity == 63 and a.max_blocks == 25
    ctx = [0] * 6
    for _ in range(3000):
        s = rng.randrange(6)
        op = rng.random()
        if op < 0.6:
            want = min(400, ctx[s] + rng.choice([1, 1, 1, 16, 37, 120]))
            before = (a.n_blocks[s], a.free_blocks)
            if a.can_fit(s, want):
                a.ensure(s, want)
                ctx[s] = want
            else:
                with pytest.raises(MemoryError):
                    a.ensure(s, want)
                assert (a.n_blocks[s], a.free_blocks) == before
        elif op < 0.75:
            a.release(s)
            ctx[s] = 0
        owned = [b for k in range(6) for b in a.blocks_of(k).tolist()]
        assert len(owned) == len(set(owned)) and 0 not in owned and len(owned) + a.free_blocks == a.capacity
        assert all(a.n_blocks[k] == a.blocks_for(ctx[k]) for k in range(6))
        assert all(int(a.table[k, a.n_blocks[k]:].abs().sum()) == 0 for k in range(6))
    with pytest.raises(MemoryError):
        a.ensure(0, 401)                                             # longer than a table row
    for k in range(6):
        a.release(k)
    assert a.free_blocks == a.capacity and int(a.table.abs().sum()) == 0


def _stub_kernels(monkeypatch, calls):
    """Replaces this package's kernel entry points with recorders, so that the engines' Python (buffers, call order, options)
    runs on a machine without a GPU."""
    import skygdr_b200.ops as ops

    class Attn:
        def __init__(self, *a, **k):
            self.status = torch.zeros(4, dtype=torch.int32)
            self.kw = k

        def __call__(self, q, pool, li, table, ctx, max_ctx=None, out=None):
            calls.append("attn")
            return out

    def shaped(name, a, k):
        """What the real op returns when no output buffer is passed: a tensor of the right shape."""
        if name == "embedding":
            return torch.zeros((a[0].numel(), a[1].shape[1]), dtype=torch.bfloat16)
        if name == "rmsnorm":
            return torch.zeros_like(a[0])
        if name == "gemm":
            return torch.zeros((a[0].shape[0], a[1].shape[0] // (2 if k.get("gated") else 1)), dtype=torch.bfloat16)
        if name == "rope_append":
            return torch.zeros((a[0].shape[0], a[8], 128), dtype=torch.bfloat16)      # q: [tokens][q_heads][128]
        return None

    def rec(name):
        def f(*a, **k):
            calls.append((name, {x: (v if isinstance(v, (bool, int, float, str)) else "tensor") for x, v in k.items() if x not in ("out", "q_out") and v is not None}))
            out = k.get("out", k.get("q_out"))
            return out if out is not None else shaped(name, a, k)
        return f

    class Prefill:
        def __init__(self, dev, *a, **k):
            pass

        def __call__(self, q, pool, li, table, seq_start, max_len, out=None, pos0=None):
            calls.append(("prefill_attn", {"pos0": pos0.tolist(), "seq_start": seq_start.tolist(), "rows": table.shape[0], "max_len": max_len}))
            return out

    monkeypatch.setattr(ops, "PagedAttention", Attn)
    monkeypatch.setattr(ops, "PrefillAttention", Prefill)
    for name in ("embedding", "rmsnorm", "gemm", "rope_append", "argmax", "sample", "silu_mul"):
        monkeypatch.setattr(ops, name, rec(name))
    monkeypatch.setattr(ops, "rope_inv_freq", lambda theta, dev, D: torch.ones(D // 2))


def test_decode_engine_issues_the_expected_kernel_sequence(monkeypatch):
    """The decode engine's host side with the kernels stubbed out: a step is embedding, eight kernels per layer, final norm,
    lm_head, argmax; a positive temperature swaps argmax for the sampling kernel keyed by the positions."""
    from skygdr_b200 import ops
    from skygdr_b200.models import Qwen3Config, Qwen3Decoder, Qwen3Weights

    calls = []
    _stub_kernels(monkeypatch, calls)
    cfg = Qwen3Config.tiny(layers=2)
    pool = ops.PagedKVPool(cfg.geometry, 8, "hnd", device="cpu")
    eng = Qwen3Decoder(cfg, Qwen3Weights(cfg, "cpu", seed=0), pool, max_batch=2, max_ctx=64, attn_chunk=64)
    eng.set_batch(torch.tensor([1, 2], dtype=torch.int32), torch.tensor([3, 4], dtype=torch.int32), torch.zeros((2, 4), dtype=torch.int32))
    assert eng.ctx_lens.tolist() == [4, 5]
    out = eng.step(max_ctx=64)
    names = [c if isinstance(c, str) else c[0] for c in calls]
    layer = ["rmsnorm", "gemm", "rope_append", "attn", "gemm", "rmsnorm", "gemm", "gemm"]
    assert names == ["embedding"] + layer * 2 + ["rmsnorm", "gemm", "argmax"] and len(names) == eng.kernels_per_step
    assert out.shape == (2,) and eng.positions.tolist() == [4, 5] and eng.ctx_lens.tolist() == [5, 6]      # the step advanced the batch
    assert [c[1].get("gated", False) for c in calls if not isinstance(c, str) and c[0] == "gemm"] == [False, False, True, False] * 2 + [False]
    calls.clear()
    eng.temperature, eng.sample_seed = 0.7, 5
    eng.step(max_ctx=64)
    assert calls[-1][0] == "sample" and calls[-1][1] == {"positions": "tensor"}


def test_prefill_issues_the_expected_kernel_sequence(monkeypatch):
    """The prefill path's host side with the kernels stubbed out: per layer norm, QKV, RoPE + append, the prefill attention
    kernel, O, norm, gate/up, down; logits only for each prompt's last token. With a chunk smaller than the prompts the stack
    runs once per pass, and a prompt that continues in a later pass tells the attention kernel how many tokens precede it."""
    from skygdr_b200 import ops
    from skygdr_b200.models import Qwen3Config, Qwen3Decoder, Qwen3Weights

    calls = []
    _stub_kernels(monkeypatch, calls)
    cfg = Qwen3Config.tiny(layers=2)
    pool = ops.PagedKVPool(cfg.geometry, 64, "hnd", device="cpu")
    eng = Qwen3Decoder(cfg, Qwen3Weights(cfg, "cpu", seed=0), pool, max_batch=2, max_ctx=512, attn_chunk=128)
    table = torch.arange(2 * 32, dtype=torch.int32).view(2, 32)
    seq_lens = [20, 9]
    logits = eng.prefill(torch.randint(0, cfg.vocab, (sum(seq_lens),)), seq_lens, table)
    assert logits.shape == (2, cfg.vocab)
    names = [c if isinstance(c, str) else c[0] for c in calls]
    layer = ["rmsnorm", "gemm", "rope_append", "prefill_attn", "gemm", "rmsnorm", "gemm", "gemm"]
    assert names == ["embedding"] + layer * 2 + ["rmsnorm", "gemm"]
    assert [c[1] for c in calls if c[0] == "prefill_attn"][0] == {"pos0": [0, 0], "seq_start": [0, 20, 29], "rows": 2, "max_len": 20}
    # the plan: passes of at most `chunk` tokens, a sequence at most once per pass, pieces in order
    assert Qwen3Decoder.prefill_plan([20, 9], 16) == [[(0, 0, 16)], [(0, 16, 20), (1, 0, 9)]]
    assert Qwen3Decoder.prefill_plan([5, 40, 3], 16) == [[(0, 0, 5), (1, 0, 11)], [(1, 11, 27)], [(1, 27, 40), (2, 0, 3)]]
    assert Qwen3Decoder.prefill_plan([8], 8) == [[(0, 0, 8)]]
    calls.clear()
    logits = eng.prefill(torch.randint(0, cfg.vocab, (sum(seq_lens),)), seq_lens, table, chunk=16)
    assert logits.shape == (2, cfg.vocab)
    names = [c if isinstance(c, str) else c[0] for c in calls]
    assert names == (["embedding"] + layer * 2) * 2 + ["rmsnorm", "gemm"]               # two passes through the stack, one lm_head
    attn = [c[1] for c in calls if c[0] == "prefill_attn"]
    assert attn[0] == {"pos0": [0], "seq_start": [0, 16], "rows": 1, "max_len": 16}
    assert attn[2] == {"pos0": [16, 0], "seq_start": [0, 4, 13], "rows": 2, "max_len": 9}


class _FakeHeap:
    """Stand-in for the CUDA IPC symmetric heap: local tensors on the CPU, made-up peer addresses (rank in the high bits)."""

    def __init__(self, nbytes, rank, world, device, group=None):
        self.rank, self.world, self.off, self.names = rank, world, 0, {}

    def alloc(self, name, nbytes, align=256, local=True):
        self.off = (self.off + align - 1) // align * align
        self.names[name] = (self.off, nbytes)
        self.off += nbytes
        return self.names[name][0]

    def ptr(self, name, rank, byte_offset=0):
        return (rank + 1 << 40) + self.names[name][0] + byte_offset

    def all_ptrs(self, name, byte_offset=0):
        return [self.ptr(name, r, byte_offset) for r in range(self.world)]

    def local_tensor(self, name, shape, dtype):
        return torch.zeros(shape, dtype=dtype)


@pytest.mark.parametrize("collective", ["rs_ag", "oneshot"])
def test_tensor_parallel_engine_issues_the_expected_kernel_sequence(monkeypatch, collective):
    """The tensor-parallel engine's host side with heap and kernels stubbed out, for both collective forms: kernels per step,
    which GEMMs wait for an all-gather or push a reduce-scatter / one-shot all-reduce, the (step, use) counters they are given,
    and that the expected arrival counts match what the pushing GEMMs' tile counts produce."""
    import skygdr_b200.parallel.tp as tp
    from skygdr_b200 import ops
    from skygdr_b200.models import Qwen3Config, Qwen3Weights

    calls = []
    _stub_kernels(monkeypatch, calls)
    monkeypatch.setattr(tp, "SymmetricHeap", _FakeHeap)
    monkeypatch.setattr(tp, "new_status", lambda dev: torch.zeros(16, dtype=torch.int32))
    import sys

    monkeypatch.setattr(sys.modules["skygdr_b200.ops.gemm"], "new_status", lambda dev: torch.zeros(16, dtype=torch.int32))
    monkeypatch.setattr(tp.dist, "barrier", lambda group=None: None)

    class Rec:
        def __getattr__(self, name):
            def f(*a, **k):
                if name in ("gemm_workspace_floats", "gemm_counter_count"):      # sizing helpers of split-K, not launches
                    return 1024
                calls.append((name, a, k))
                return 0
            return f

    world, rank = 2, 1
    cfg = Qwen3Config.tiny(layers=2)
    cfg.q_heads, cfg.kv_heads, cfg.ffn, cfg.vocab = 8, 4, 512, 600
    w = Qwen3Weights(cfg, "cpu", seed=0, tp_rank=rank, tp_world=world)
    pool = ops.PagedKVPool(ops.KVGeometry(cfg.layers, cfg.kv_heads // world, cfg.head_dim), 8, "hnd", device="cpu")
    B = 4
    eng = tp.TPDecoder(cfg, w, pool, B, 64, rank, world, attn_chunk=128, collective=collective)
    eng._C = Rec()
    eng.set_batch(torch.arange(B, dtype=torch.int32), torch.full((B,), 5, dtype=torch.int32), torch.zeros((B, 4), dtype=torch.int32))
    eng.step(max_ctx=64)
    names = [c if isinstance(c, str) else c[0] for c in calls]
    layer = ["tp_norm", "gemm_tp", "rope_append", "attn", "gemm_tp", "tp_norm", "gemm_tp", "gemm_tp"]
    assert names == ["embedding"] + layer * 2 + ["tp_norm", "gemm_tp", "tp_argmax", "step_increment"]
    assert len(names) == eng.kernels_per_step
    gemms = [c for c in calls if not isinstance(c, str) and c[0] == "gemm_tp"]
    # gemm_tp(x, w, y, splits, gated, ws, counters, status, ag, rs, ntok)
    ag = [bool(g[1][8]) for g in gemms]
    rs = [bool(g[1][9]) for g in gemms]
    assert rs == [False, True, False, True] * 2 + [False]                       # O and down push their partial tiles
    if collective == "rs_ag":
        assert ag == [True, False, True, False] * 2 + [True]                    # QKV, gate/up and lm_head wait for gathered rows
        uses = [(g[1][8][3], g[1][8][4]) for g in gemms if g[1][8]]             # (uses per step, use index)
        assert uses == [(3, 0), (2, 0), (3, 1), (2, 1), (3, 2)]
        assert all(len(g[1][9]) == 5 for g in gemms if g[1][9])                 # world, src rank, rows per rank, dst ptrs, counter ptrs
    else:
        assert not any(ag)                                                       # activations are replicated: nobody waits in a GEMM
        pushes = [g[1][9] for g in gemms if g[1][9]]
        assert all(p[0] == world and p[1] == rank and p[2] == B and p[5] is True for p in pushes)      # slot [this rank][row], to everybody
        assert eng.resid.shape[0] == B                                           # replicated residual stream
    norms = [c for c in calls if not isinstance(c, str) and c[0] == "tp_norm"]
    # tp_norm(rs_buf, rs_ctr, seq, resid, w, ag_dst, ag_ctr, rank, eps, timeout, status[, rs_world=])
    seqs = [n[1][2] for n in norms]
    assert seqs[0] == () and [s[1:3] for s in seqs[1:]] == [(2, 0), (2, 0), (2, 1), (2, 1)]       # (uses per step, use index) of rs0 / rs1
    tiles_h = (cfg.hidden + 127) // 128
    for s in seqs[1:]:
        assert s[3] % (world * tiles_h) == 0 and s[3] >= world * tiles_h        # arrivals: every output tile of every rank's GEMM
    if collective == "oneshot":
        assert all(n[2].get("rs_world") == world for n in norms) and all(n[1][6] == [0] for n in norms)   # local destination, no arrival


def test_paged_attention_wrapper_sizes_scratch_and_passes_the_bounds(monkeypatch):
    """The Python face of the decode attention with the launch stubbed out: scratch sizes, and what reaches the extension: the
    max_ctx of the call cut to what the engine and the block-table row cover, the tensor map's row count for the tensor-core
    kernel, and the pool's block count that the CUDA-core kernel checks block ids against."""
    import sys

    from skygdr_b200 import ops

    att = sys.modules["skygdr_b200.ops.attention"]            # loaded by the import of ops above
    monkeypatch.setattr(att, "new_status", lambda dev: torch.zeros(16, dtype=torch.int32))
    seen = {}

    class C:
        @staticmethod
        def paged_attn_decode(*a, **k):
            seen["args"], seen["kw"] = a, k

    pool = ops.PagedKVPool(ops.KVGeometry(layers=2, kv_heads=2), 8, "hnd", device="cpu")
    q = torch.zeros((3, 4, 128), dtype=torch.bfloat16)
    table, ctx = torch.zeros((3, 8), dtype=torch.int32), torch.tensor([5, 40, 64], dtype=torch.int32)
    a = ops.PagedAttention("cpu", 3, 4, 2, max_ctx=2300, chunk_tokens=512, impl="tc")
    a._C = C
    assert a.max_splits == 5 and a.part_o.shape == (3, 4, 5, 128) and a.part_m.shape == (3, 4, 5)
    out = a(q, pool, 1, table, ctx, max_ctx=100)
    assert out.shape == q.shape and seen["kw"] == {"num_blocks": 8}
    assert seen["args"][9] == 100 and seen["args"][10] == 512                  # max_ctx of this call, chunk size
    assert seen["args"][-1] == (pool.data.numel() - 1 * pool.strides[1]) // 128     # rows from this layer's first page to the end
    a(q, pool, 1, table, ctx, max_ctx=1000)
    assert seen["args"][9] == 8 * 16                                           # a table row of 8 blocks covers 128 tokens, no more
    simt = ops.PagedAttention("cpu", 3, 4, 2, max_ctx=2300, chunk_tokens=500, impl="simt")
    simt._C = C
    simt(q, pool, 0, torch.zeros((3, 200), dtype=torch.int32), ctx)
    assert seen["kw"] == {"num_blocks": 8} and seen["args"][-1] == 0 and seen["args"][9] == 2300
    with pytest.raises(AssertionError):
        ops.PagedAttention("cpu", 3, 4, 2, max_ctx=2300, chunk_tokens=500, impl="tc")       # whole key tiles of 128 tokens


def test_gemm_wrapper_argument_order_matches_the_extension(monkeypatch):
    """ops.gemm with the launch stubbed out: which positional arguments reach the extension for the plain, split-K and persistent
    forms, and that many-token shapes take the persistent form on their own. The binding's own signature is read from the built
    module, so a mismatch in count shows here."""
    import sys

    import skygdr_b200.ops  # noqa: F401  (makes sure the submodule is loaded; its name in the package is shadowed by the function)
    from skygdr_b200._ext import load

    g = sys.modules["skygdr_b200.ops.gemm"]
    monkeypatch.setattr(g, "new_status", lambda dev: torch.zeros(16, dtype=torch.int32))
    monkeypatch.setattr(g, "_sms", lambda dev: 148)
    g._WS.clear()
    sig = load().gemm.__doc__
    names = ["x", "w", "y", "splits", "gated", "workspace", "counters", "status", "ntok", "persistent"]
    assert all(f"{n}:" in sig for n in names) and [sig.index(f"{a}:") < sig.index(f"{b}:") for a, b in zip(names, names[1:])] == [True] * 9
    seen = []

    class C:
        gemm_workspace_floats = staticmethod(lambda *a: 4096)
        gemm_counter_count = staticmethod(lambda *a: 64)
        gemm = staticmethod(lambda *a: seen.append(a))

    monkeypatch.setattr(g, "load", lambda: C)
    x, w = torch.zeros((16, 1024), dtype=torch.bfloat16), torch.zeros((512, 1024), dtype=torch.bfloat16)
    y = g.gemm(x, w)
    a = seen[-1]
    assert y.shape == (16, 512) and len(a) == 9 and a[3] >= 1 and a[4] is False
    g.gemm(x, w, splits=4, ntok=16)
    a = seen[-1]
    assert a[3] == 4 and a[5] is not None and a[6] is not None and a[8] == 16
    big = torch.zeros((700, 1024), dtype=torch.bfloat16)
    g.gemm(big, w)                                                             # more than 256 tokens: persistent on its own
    a = seen[-1]
    assert len(a) == 10 and a[3] == 1 and a[8] == 256 and a[9] in (1, 2)      # 1: 128-row tiles, 2: 256 x 256 tiles
    g.gemm(big, w, persistent="wide")
    assert seen[-1][9] == 2
    g.gemm(big, w, persistent="narrow")
    assert seen[-1][9] == 1
    g.gemm(big, torch.zeros((1024, 1024), dtype=torch.bfloat16), gated=True)
    assert seen[-1][4] is True and (seen[-1][8], seen[-1][9]) in ((128, 1), (256, 2))   # gated: 128-token tiles, or two blocks per 256 tokens
    g.gemm(big, w, persistent=False)                                           # the comparison form: one tile per CTA
    assert len(seen[-1]) == 9 and seen[-1][3] == 1
    g.gemm(x, w, persistent=None)
    assert len(seen[-1]) == 9                                                  # few tokens: never persistent by default
    # the tile rule picks what was measured faster on B200 at each of these shapes
    assert [g.wide_tiles_pay(M, N, K, 148, False) for M, N, K in ((2048, 4096, 4096), (4096, 4096, 4096), (8192, 4096, 4096),
                                                                 (8192, 6144, 4096), (8192, 4096, 12288))] == [True, True, False, True, True]
    assert not g.wide_tiles_pay(2048, 151936, 4096, 148, False)                 # N not a multiple of 256
    g._WS.clear()


def test_bindings_expose_the_keywords_the_python_side_uses():
    """Keyword names that the Python wrappers pass must exist in the built extension's signatures (read from its docstrings)."""
    from skygdr_b200._ext import load

    C = load()
    for fn, words in {"paged_attn_decode": ["num_blocks:", "pool_rows:"],
                      "prefill_attn": ["pos0:"], "sample": ["temperature:", "seed:", "positions:"],
                      "gemm": ["persistent: typing.SupportsInt = 0"],
                      "tp_norm": ["rs_world:"]}.items():
        doc = getattr(C, fn).__doc__
        assert all(w in doc for w in words), (fn, doc)


def test_build_decode_engine_lays_out_pool_and_tables(monkeypatch):
    """What the benchmark calls to get an engine, with the kernels stubbed out: every sequence gets its own blocks (never block
    0), enough for its context plus the growth asked for, and the options reach the engine."""
    from skygdr_b200.models import Qwen3Config
    from skygdr_b200.parallel.tp import build_decode_engine

    calls = []
    _stub_kernels(monkeypatch, calls)
    cfg = Qwen3Config.tiny(layers=2)
    ctx = torch.tensor([40, 7, 130, 64])
    eng, table = build_decode_engine(cfg, torch.device("cpu"), 0, 1, ctx, extra_tokens=20, seed=1, attn_chunk=512)
    need = [(int(c) + 20 + 15) // 16 for c in ctx]
    used = [table[i, :need[i]].tolist() for i in range(4)]
    flat = [b for row in used for b in row]
    assert len(flat) == len(set(flat)) and 0 not in flat and max(flat) < eng.pool.num_blocks == sum(need) + 1
    assert all(int(table[i, need[i]:].abs().sum()) == 0 for i in range(4))
    assert eng.max_ctx == 130 + 20 + 1 and table.shape == (4, eng.max_blocks) and eng.max_batch == 4
    assert eng.attn.kw["impl"] == "tc"
    assert float(eng.pool.data.float().std()) > 0.5                      # N(0, 1) cache contents, as the benchmark states
    eng.set_batch(torch.zeros(4, dtype=torch.int32), ctx.int(), table)
    eng.step()
    assert len(calls) == eng.kernels_per_step


def test_attention_chunk_planner_orders_candidates_as_measured():
    """The fluid model behind the chunk planner: on the two batches where launches were timed on B200 it must put the candidates
    in the measured order (contexts 8k-16k: larger chunks faster, 512 tokens slowest; the benchmark's contexts 2k-16k: 1536 ahead
    of 1024 and 2048), and the planner must return a multiple of 128 from its candidates."""
    import torch

    from skygdr_b200.ops.attention import plan_chunk_tokens, simulate_decode_launch

    g = torch.Generator().manual_seed(0)
    long_ctx = torch.randint(8192, 16385, (16,), generator=g).tolist()
    t = {c: simulate_decode_launch(long_ctx, 8, c) for c in (512, 768, 1024, 1536, 2048)}
    assert t[512] > t[768] > t[1024] >= t[1536] > t[2048]
    g = torch.Generator().manual_seed(0)
    bench_ctx = (torch.randint(2048, 16385, (16,), generator=g) + 20).tolist()
    t = {c: simulate_decode_launch(bench_ctx, 8, c) for c in (1024, 1536, 2048)}
    assert t[1536] < t[1024] and t[1536] < t[2048]
    assert plan_chunk_tokens(bench_ctx, 8) == 1536
    assert plan_chunk_tokens([], 8) == 1024 and plan_chunk_tokens([100, 200], 8) % 128 == 0
