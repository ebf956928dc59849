"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math
import os
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import skygdr_b200.ops as ops

    from skygdr_b200._ext import load

    load()  # a missing extension is an error on a GPU box
    return ops


def _pools(ops, n_src=40, n_dst=48, layers=3, heads=8, seed=0):
    g = ops.KVGeometry(layers=layers, kv_heads=heads)
    torch.manual_seed(seed)
    src = ops.PagedKVPool(g, n_src, "nhd")
    src.data.normal_()
    dst = ops.PagedKVPool(g, n_dst, "hnd")
    return g, src, dst


@pytest.mark.parametrize("method", ["simt", "tma"])
def test_kv_transfer_exact(ops, method):
    g, src, dst = _pools(ops)
    n = 23
    sb = torch.randperm(src.num_blocks, device="cuda")[:n].int()
    db = torch.randperm(dst.num_blocks, device="cuda")[:n].int()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    flow = ops.KvTransferFlow("cuda", pages_per_chunk=4, method=method)
    flow.transfer(src, [ops.RemotePool.of(dst, flag)], sb, db)
    st = flow.result()
    assert st["status"] == 0 and st["cursor"] == 2**64 - 1
    assert st["bytes_done"] == ops.link_bytes(g, n)
    assert torch.equal(dst.data[db.long()], ops.reference_transfer(src, sb))
    assert int(flag.item()) == flow.seq
    untouched = torch.ones(dst.num_blocks, dtype=torch.bool, device="cuda")
    untouched[db.long()] = False
    assert float(dst.data[untouched].abs().sum()) == 0.0


@pytest.mark.parametrize("method", ["simt", "tma"])
def test_kv_transfer_scatter_and_replicate(ops, method):
    g, src, _ = _pools(ops, layers=2)
    gd = ops.KVGeometry(layers=2, kv_heads=2)
    parts = [ops.PagedKVPool(gd, 16, "hnd") for _ in range(4)]
    sb = torch.arange(5, 14, device="cuda").int()
    db = torch.arange(0, 9, device="cuda").int()
    flow = ops.KvTransferFlow("cuda", method=method)
    flow.transfer(src, [ops.RemotePool.of(p) for p in parts], sb, db)
    assert flow.result()["status"] == 0
    for i, p in enumerate(parts):
        assert torch.equal(p.data[db.long()], ops.reference_transfer(src, sb, slice(2 * i, 2 * i + 2)))
    full = [ops.PagedKVPool(g, 16, "hnd") for _ in range(3)]
    flow.transfer(src, [ops.RemotePool.of(p) for p in full], sb, db, replicate=True)
    st = flow.result()
    assert st["bytes_done"] == ops.link_bytes(g, 9, 3, replicate=True)
    for p in full:
        assert torch.equal(p.data[db.long()], ops.reference_transfer(src, sb))


def test_kv_transfer_fp8_pack(ops):
    from skygdr_b200.ops.kv_transfer import RemotePool, fp8_mx_reference

    g, src, _ = _pools(ops, layers=2)
    nb = 12
    q = torch.zeros((nb, g.layers, 2, g.kv_heads, 16, 128), dtype=torch.uint8, device="cuda")
    sc = torch.zeros((nb, g.layers, 2, g.kv_heads, 16, 4), dtype=torch.uint8, device="cuda")
    sb = torch.randperm(src.num_blocks, device="cuda")[:nb].int()
    db = torch.arange(nb, device="cuda").int()
    flow = ops.KvTransferFlow("cuda")
    rp = RemotePool(q.data_ptr(), (q.stride(0), q.stride(1), q.stride(2)), g.kv_heads, sc.data_ptr())
    flow.transfer(src, [rp], sb, db, fp8=True)
    assert flow.result()["status"] == 0
    want_q, want_s = fp8_mx_reference(ops.reference_transfer(src, sb))
    assert torch.equal(sc, want_s)
    # identical scales; the quantised values may differ by one rounding step where x/scale sits on a tie
    got = q.view(torch.float8_e4m3fn).float() * torch.exp2(sc.float() - 127).repeat_interleave(32, -1)
    ref = ops.reference_transfer(src, sb).float()
    assert (got - ref).abs().max() <= 0.07 * ref.abs().max()
    assert (q != want_q).float().mean() < 1e-3


@pytest.mark.parametrize("method", ["simt", "tma"])
def test_kv_transfer_credit_yield_and_resume(ops, method):
    g, src, dst = _pools(ops, layers=2)
    n = 20
    sb = torch.arange(n, device="cuda").int()
    db = torch.arange(n, device="cuda").int()
    page = ops.CreditPage(flow_id=7, unlimited=False)
    total = ops.link_bytes(g, n)
    page.grant(total // 2)                       # nothing will ever add to this: a host-made stall
    flow = ops.KvTransferFlow("cuda", page=page, pages_per_chunk=2, max_wait_ms=1.0, method=method)
    flow.transfer(src, [ops.RemotePool.of(dst)], sb, db)
    st = flow.result()
    assert st["status_name"] == "YIELD_CREDIT"
    assert 0 < st["bytes_done"] <= total // 2
    chunk_bytes = 2 * g.page_elems * 2
    assert st["cursor"] == st["bytes_done"] // chunk_bytes   # everything below the cursor is done
    assert page.read()["yields"] == 1
    page.grant(total)
    flow.resume(st)
    st2 = flow.result()
    assert st2["status"] == 0 and st["bytes_done"] + st2["bytes_done"] == total
    assert torch.equal(dst.data[db.long()], ops.reference_transfer(src, sb))
    assert page.read()["completed_bytes"] == total
    # stop flag: the kernel returns at once with STOPPED
    page.grant(total, stop=True)
    flow.transfer(src, [ops.RemotePool.of(dst)], sb, db)
    assert flow.result()["status_name"] == "STOPPED"


@pytest.mark.parametrize("method", ["simt", "tma"])
def test_kv_transfer_rejects_block_ids_outside_the_pools(ops, method):
    """A corrupted block list (made on the host) never becomes an out-of-range access: the kernel checks every block id
    against the pool sizes, skips the page, and reports BAD_INDEX with the position of the offending pair."""
    g, src, dst = _pools(ops, layers=2)
    dst.data.fill_(-2.0)
    sb = torch.tensor([3, 5, 7, 9], device="cuda").int()
    db = torch.tensor([0, 1, 2, 3], device="cuda").int()
    for bad_src, bad_dst, where in ((1000, 1, 1), (5, 48, 1), (-1, 2, 2)):
        sb2, db2 = sb.clone(), db.clone()
        sb2[where], db2[where] = bad_src, bad_dst
        flow = ops.KvTransferFlow("cuda", pages_per_chunk=4, method=method)
        flow.transfer(src, [ops.RemotePool.of(dst)], sb2, db2)
        st = flow.result()
        assert st["status_name"] == "BAD_INDEX" and st["detail"] == where, st
    assert bool((dst.data[4:] == -2.0).all())                     # nothing beyond the named destination blocks was written
    flow = ops.KvTransferFlow("cuda", method=method)              # and a clean list still goes through
    flow.transfer(src, [ops.RemotePool.of(dst)], sb, db)
    assert flow.result()["status"] == 0
    assert torch.equal(dst.data[db.long()], ops.reference_transfer(src, sb))


@pytest.mark.parametrize("policy", ["stall", "unpaced", "static"])
def test_kv_transfer_follows_the_page_when_the_control_side_goes_silent(ops, policy):
    """Nothing renews the grant (a control side that died: made on the host by simply not granting). The kernel waits
    for credit, sees the epoch stand still for 5 windows of 1 ms, and follows the page's dead policy; every wait is bounded."""
    g, src, dst = _pools(ops, layers=2)
    n = 20
    sb = torch.arange(n, device="cuda").int()
    db = torch.arange(n, device="cuda").int()
    total = ops.link_bytes(g, n)
    page = ops.CreditPage(flow_id=9, unlimited=False)
    page.set_heartbeat(window_ms=1.0, dead_after_windows=5, policy=policy, fallback_gbps=total / 1e9 / 0.004)   # static: all of it in 4 windows
    page.grant(total // 4)
    flow = ops.KvTransferFlow("cuda", page=page, pages_per_chunk=2, max_wait_ms=200.0, method="simt")
    t0 = time.perf_counter()
    flow.transfer(src, [ops.RemotePool.of(dst)], sb, db)
    st = flow.result()
    wall = time.perf_counter() - t0
    rd = page.read()
    assert rd["heartbeat_lost"] == rd["epoch"] + 1                # the data path flagged the silence in the page
    assert wall < 0.15                                            # decided after ~5 ms, far below the 200 ms credit wait
    if policy == "stall":
        assert st["status_name"] == "CONTROL_LOST" and 0 < st["bytes_done"] <= total // 4
        page.grant(total)                                         # the control side is back: resume from the cursor
        flow.resume(st)
        st2 = flow.result()
        assert st2["status"] == 0 and st["bytes_done"] + st2["bytes_done"] == total
    else:
        assert st["status"] == 0 and st["bytes_done"] == total
    assert torch.equal(dst.data[db.long()], ops.reference_transfer(src, sb))


def test_kv_offload_to_mapped_host(ops):
    from skygdr_b200._ext import load
    from skygdr_b200.ops.kv_transfer import RemotePool

    C = load()
    g, src, _ = _pools(ops, layers=2)
    nb = 6
    nbytes = nb * g.block_elems * 2
    hptr, dptr = C.host_alloc_mapped(nbytes)
    try:
        sb = torch.tensor([3, 9, 1, 30, 7, 22], device="cuda").int()
        db = torch.arange(nb, device="cuda").int()
        flow = ops.KvTransferFlow("cuda", ctas=16)
        s = src.strides
        flow.transfer(src, [RemotePool(dptr, s, g.kv_heads)], sb, db, keep_layout=True)
        assert flow.result()["status"] == 0
        import ctypes

        host = torch.frombuffer((ctypes.c_char * nbytes).from_address(hptr), dtype=torch.bfloat16).view(nb, -1)
        assert torch.equal(host, src.data[sb.long()].cpu().view(nb, -1))
    finally:
        C.host_free_mapped(hptr)


@pytest.mark.parametrize("op", ["read", "write", "rw", "copy", "axpy"])
def test_memhog_ops(ops, op):
    hog = ops.Memhog("cuda", gb=0.25, op=op, chunk_bytes=1 << 18)
    hog.a.copy_(torch.arange(hog.a.numel(), device="cuda") % 7)
    if op == "axpy":
        hog.b.fill_(1.0)
    hog.launch(iters=2, alpha=0.5)
    st = hog.result()
    assert st["status"] == 0 and st["bytes_done"] == 2 * hog.bytes_per_pass()
    if op == "read":
        assert abs(float(hog.sink.item()) - 2 * float(hog.a.double().sum())) < 1e-3 * float(hog.a.double().sum())
    if op == "copy":
        assert torch.equal(hog.a, hog.b)
    if op == "axpy":
        assert torch.allclose(hog.b, 1.0 + 2 * 0.5 * hog.a)
    if op == "rw":
        assert torch.allclose(hog.b, hog.a * 1.0001 + 0.5)


def test_memhog_duty_cycle_and_time_limit(ops):
    hog = ops.Memhog("cuda", gb=0.5, op="copy")
    hog.launch(iters=0, seconds=0.05)
    full = hog.result()
    assert 0.04 < full["seconds"] < 0.2
    hog.launch(iters=0, seconds=0.05, duty_on_ms=1.0, duty_off_ms=1.0)
    half = hog.result()
    assert 0.3 < half["bytes_done"] / full["bytes_done"] < 0.75


@pytest.mark.parametrize("impl", ["simt", "tc"])
@pytest.mark.parametrize("kv_heads,q_heads", [(8, 32), (1, 4), (2, 4), (4, 4), (1, 8)])
def test_paged_attention_matches_reference(ops, kv_heads, q_heads, impl):
    torch.manual_seed(1)
    g = ops.KVGeometry(layers=2, kv_heads=kv_heads)
    ctx = torch.tensor([1, 15, 16, 17, 511, 512, 513, 1300, 2049, 64], dtype=torch.int32, device="cuda")
    B = ctx.numel()
    max_blocks = (int(ctx.max()) + 15) // 16
    nblk = int(((ctx + 15) // 16).sum()) + 4
    pool = ops.PagedKVPool(g, nblk, "hnd")
    pool.data.normal_()
    perm = torch.randperm(nblk, device="cuda").int()
    table = torch.zeros((B, max_blocks), dtype=torch.int32, device="cuda")
    o = 0
    for b in range(B):
        nb = (int(ctx[b]) + 15) // 16
        table[b, :nb] = perm[o:o + nb]
        o += nb
    q = torch.randn((B, q_heads, 128), dtype=torch.bfloat16, device="cuda")
    attn = ops.PagedAttention("cuda", B, q_heads, kv_heads, max_ctx=4096, chunk_tokens=512, impl=impl)
    for layer in (0, 1):
        out = attn(q, pool, layer, table, ctx, max_ctx=int(ctx.max()))
        ref = ops.paged_attn_reference(q, pool, layer, table, ctx)
        torch.cuda.synchronize()
        assert ops.read_status(attn.status)["status"] == 0
        assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), float((out.float() - ref).abs().max())
    # counters are left at zero for the next launch
    assert int(attn.counters.abs().sum()) == 0


@pytest.mark.parametrize("impl", ["simt", "tc"])
def test_paged_attention_reports_lengths_and_block_ids_it_cannot_trust(ops, impl):
    """A context length beyond max_ctx is cut to it and reported (the split count the combine waits for stays inside the
    grid, so the self-resetting counters end at zero); a block id outside the pool is reported and never dereferenced."""
    torch.manual_seed(3)
    g = ops.KVGeometry(layers=1, kv_heads=2)
    ctx = torch.tensor([300, 520, 77], dtype=torch.int32, device="cuda")
    mb = (520 + 15) // 16
    pool = ops.PagedKVPool(g, 3 * mb + 2, "hnd")
    pool.data.normal_()
    table = (torch.randperm(3 * mb, device="cuda") + 1).int().view(3, mb).contiguous()
    q = torch.randn((3, 8, 128), dtype=torch.bfloat16, device="cuda")
    ref = ops.paged_attn_reference(q, pool, 0, table, ctx)
    attn = ops.PagedAttention("cuda", 3, 8, 2, max_ctx=520, chunk_tokens=256, impl=impl)
    bad_ctx = ctx.clone()
    bad_ctx[1] = 9000
    out = attn(q, pool, 0, table, bad_ctx, max_ctx=520)
    torch.cuda.synchronize()
    st = ops.read_status(attn.status)
    assert st["status_name"] == "BAD_INDEX" and st["detail"] == (0x40000000 | 1)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    assert int(attn.counters.abs().sum()) == 0
    if impl == "simt":                                      # the tensor-core kernel's loads are bounded by its tensor map instead
        attn2 = ops.PagedAttention("cuda", 3, 8, 2, max_ctx=520, chunk_tokens=256, impl=impl)
        bad_table = table.clone()
        bad_table[2, 1] = 1 << 20
        out = attn2(q, pool, 0, bad_table, ctx, max_ctx=520)
        torch.cuda.synchronize()
        st = ops.read_status(attn2.status)
        assert st["status_name"] == "BAD_INDEX" and st["detail"] == ((2 << 16) | 1)
        assert torch.allclose(out[:2].float(), ref[:2], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("layout", ["hnd", "nhd"])
@pytest.mark.parametrize("kv_heads,q_heads", [(8, 32), (2, 4), (1, 1)])
def test_prefill_attention_matches_reference(ops, layout, kv_heads, q_heads):
    """Causal attention of packed prompts read in place from the paged pool, against fp32 softmax attention in PyTorch.
    Lengths straddle the 128-token tile (1, 127, 128, 129), the page (16) and several key tiles (700)."""
    torch.manual_seed(4)
    g = ops.KVGeometry(layers=2, kv_heads=kv_heads)
    lens = [1, 127, 128, 129, 300, 700, 16, 17, 256, 257, 385]
    nblk = sum((n + 15) // 16 for n in lens) + 3
    pool = ops.PagedKVPool(g, nblk, layout)
    pool.data.normal_()
    max_blocks = ((max(lens) + 127) // 128) * 8 + 8
    perm = (torch.randperm(nblk - 1, device="cuda") + 1).int()
    table = torch.zeros((len(lens), max_blocks), dtype=torch.int32, device="cuda")
    o = 0
    for s, n in enumerate(lens):
        nb = (n + 15) // 16
        table[s, :nb] = perm[o:o + nb]
        o += nb
    T = sum(lens)
    q = torch.randn((T, q_heads, 128), dtype=torch.bfloat16, device="cuda")
    seq_start = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32, device="cuda")
    attn = ops.PrefillAttention("cuda")
    for layer in (0, 1):
        out = attn(q, pool, layer, table, seq_start, max(lens))
        torch.cuda.synchronize()
        assert ops.read_status(attn.status)["status"] == 0, ops.read_status(attn.status)
        ref = ops.prefill_attn_reference(q, pool, layer, table, lens)
        err = (out.float() - ref).abs().max()
        assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), float(err)
    # the next piece of every prompt: queries start pos0 tokens into the sequence (on and off the 128-token tile and the
    # 16-token page) and attend to everything before them as well
    pos0 = [1, 127, 128, 129, 300, 700, 16, 17, 256, 257, 385]
    tails = [200, 1, 128, 130, 77, 260, 16, 300, 129, 5, 127]
    table2 = torch.zeros((len(lens), ((max(p + t for p, t in zip(pos0, tails)) + 127) // 128) * 8 + 8), dtype=torch.int32, device="cuda")
    nblk2 = sum((p + t + 15) // 16 for p, t in zip(pos0, tails)) + 3
    pool2 = ops.PagedKVPool(g, nblk2, layout)
    pool2.data.normal_()
    perm2 = (torch.randperm(nblk2 - 1, device="cuda") + 1).int()
    o = 0
    for s_, (p_, t_) in enumerate(zip(pos0, tails)):
        nb = (p_ + t_ + 15) // 16
        table2[s_, :nb] = perm2[o:o + nb]
        o += nb
    q2 = torch.randn((sum(tails), q_heads, 128), dtype=torch.bfloat16, device="cuda")
    start2 = torch.tensor([0] + list(torch.tensor(tails).cumsum(0).tolist()), dtype=torch.int32, device="cuda")
    out = attn(q2, pool2, 1, table2, start2, max(tails), pos0=torch.tensor(pos0, dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    assert ops.read_status(attn.status)["status"] == 0, ops.read_status(attn.status)
    ref = ops.prefill_attn_reference(q2, pool2, 1, table2, tails, pos0=pos0)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), float((out.float() - ref).abs().max())


@pytest.mark.parametrize("M,N,K,splits", [(16, 256, 512, 1), (16, 6144, 4096, 4), (13, 384, 1024, 2), (64, 512, 4096, 1),
                                          (128, 4096, 1536, 3), (300, 1024, 2048, 1), (32, 18992, 512, 1)])
def test_gemm_matches_reference(ops, M, N, K, splits):
    torch.manual_seed(2)
    x = torch.randn((M, K), dtype=torch.bfloat16, device="cuda")
    w = (torch.randn((N, K), dtype=torch.bfloat16, device="cuda") / math.sqrt(K)).contiguous()
    y = ops.gemm(x, w, splits=splits)
    ref = x.float() @ w.float().t()
    torch.cuda.synchronize()
    from skygdr_b200.ops.gemm import workspace_for

    assert ops.read_status(workspace_for("cuda").status)["status"] == 0
    err = (y.float() - ref).abs().max()
    assert err < 2e-2 * max(1.0, float(ref.abs().max())), float(err)


@pytest.mark.parametrize("M,F,K,splits", [(16, 512, 1024, 1), (16, 1536, 4096, 4), (100, 256, 512, 1)])
def test_gemm_gated_matches_reference(ops, M, F, K, splits):
    torch.manual_seed(3)
    x = torch.randn((M, K), dtype=torch.bfloat16, device="cuda")
    w = (torch.randn((2 * F, K), dtype=torch.bfloat16, device="cuda") / math.sqrt(K)).contiguous()
    y = ops.gemm(x, w, gated=True, splits=splits)
    gu = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    err = (y.float() - ref).abs().max()
    assert err < 2e-2 * max(1.0, float(ref.abs().max())), float(err)


@pytest.mark.parametrize("M,N,K,gated,ntok,splits", [
    (128, 768, 4096, False, 128, 8), (128, 768, 4096, False, 64, 4), (128, 4096, 1536, False, 128, 4), (128, 1536, 4096, True, 128, 8),
    (16, 6144, 4096, False, 16, 4), (16, 12288, 4096, True, 16, 2), (32, 4096, 6144, False, 32, 6), (100, 1000, 512, False, 64, 3),
    (37, 256, 1024, True, 64, 5), (3, 130, 2048, False, 16, 7), (256, 512, 2048, False, 256, 8)])
def test_gemm_cluster_split_matches_reference(ops, M, N, K, gated, ntok, splits):
    """Split-K inside a thread-block cluster (partials summed through distributed shared memory): every token tile width, splits
    that do and do not divide the tile and the K range, the gated epilogue, row and column tails; against fp32 PyTorch and
    against the workspace form of the same split."""
    torch.manual_seed(5)
    x = torch.randn((M, K), dtype=torch.bfloat16, device="cuda")
    w = (torch.randn(((2 if gated else 1) * N, K), dtype=torch.bfloat16, device="cuda") / math.sqrt(K)).contiguous()
    y = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm(x, w, out=y, gated=gated, splits=splits, ntok=ntok, cluster=True)
    ref = x.float() @ w.float().t()
    if gated:
        ref = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:]
    torch.cuda.synchronize()
    from skygdr_b200.ops.gemm import workspace_for

    assert ops.read_status(workspace_for("cuda").status)["status"] == 0
    err = (y.float() - ref).abs().max()
    assert err < 2e-2 * max(1.0, float(ref.abs().max())), float(err)
    y2 = ops.gemm(x, w, gated=gated, splits=splits, ntok=ntok)
    assert (y.float() - y2.float()).abs().max() <= 2e-2 * max(1.0, float(ref.abs().max()))


def test_rmsnorm_and_residual(ops):
    torch.manual_seed(4)
    x = torch.randn((37, 4096), dtype=torch.bfloat16, device="cuda")
    w = torch.randn((4096,), dtype=torch.bfloat16, device="cuda")
    y = ops.rmsnorm(x, w, 1e-6)
    xf = x.float()
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert torch.allclose(y.float(), ref, atol=2e-2, rtol=2e-2)
    res = torch.randn_like(x)
    res0 = res.clone()
    y2 = ops.rmsnorm(x, w, 1e-6, residual=res)
    s = (x.float() + res0.float()).bfloat16()
    assert torch.equal(res, s)
    sf = s.float()
    ref2 = sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert torch.allclose(y2.float(), ref2, atol=2e-2, rtol=2e-2)


def test_rope_qknorm_append(ops):
    torch.manual_seed(5)
    Hq, Hkv, B = 32, 8, 9
    g = ops.KVGeometry(layers=1, kv_heads=Hkv)
    pool = ops.PagedKVPool(g, 64, "hnd")
    pos = torch.tensor([0, 1, 15, 16, 100, 4095, 40000, 65535, 7], dtype=torch.int32, device="cuda")
    max_blocks = 65536 // 16
    table = torch.zeros((B, max_blocks), dtype=torch.int32, device="cuda")
    for b in range(B):
        table[b, int(pos[b]) // 16] = b * 3 + 1
    qkv = torch.randn((B, (Hq + 2 * Hkv) * 128), dtype=torch.bfloat16, device="cuda")
    qn = torch.rand(128, device="cuda").bfloat16() + 0.5
    kn = torch.rand(128, device="cuda").bfloat16() + 0.5
    inv = ops.rope_inv_freq(1e6, "cuda")
    q = ops.rope_append(qkv, qn, kn, pool, 0, inv, table, pos, Hq)

    def norm(x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).bfloat16().float()

    def rope(x, p):
        ang = p.float()[:, None, None] * inv[None, None, :]
        c, s = torch.cos(ang.double()).float(), torch.sin(ang.double()).float()
        x1, x2 = x[..., :64], x[..., 64:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    h = qkv.view(B, Hq + 2 * Hkv, 128)
    q_ref = rope(norm(h[:, :Hq], qn), pos)
    k_ref = rope(norm(h[:, Hq:Hq + Hkv], kn), pos)
    v_ref = h[:, Hq + Hkv:].float()
    assert torch.allclose(q.float(), q_ref, atol=3e-2, rtol=3e-2), float((q.float() - q_ref).abs().max())
    for b in range(B):
        blk, slot = b * 3 + 1, int(pos[b]) % 16
        assert torch.allclose(pool.data[blk, 0, 0, :, slot].float(), k_ref[b], atol=3e-2, rtol=3e-2)
        assert torch.equal(pool.data[blk, 0, 1, :, slot].float(), v_ref[b])


def test_silu_embedding_argmax(ops):
    torch.manual_seed(6)
    gu = torch.randn((21, 2 * 1536), dtype=torch.bfloat16, device="cuda")
    y = ops.silu_mul(gu)
    ref = torch.nn.functional.silu(gu[:, :1536].float()) * gu[:, 1536:].float()
    assert torch.allclose(y.float(), ref, atol=2e-2, rtol=2e-2)
    table = torch.randn((1000, 512), dtype=torch.bfloat16, device="cuda")
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device="cuda")
    assert torch.equal(ops.embedding(ids, table), table[ids.long()])
    logits = torch.randn((7, 151936), dtype=torch.bfloat16, device="cuda")
    logits[3, 77] = 100.0
    logits[3, 50000] = 100.0
    got = ops.argmax(logits)
    assert torch.equal(got.long(), logits.float().argmax(-1)) or int(got[3]) == 77
    assert int(got[3]) == 77


def test_peer_wait_runs_out_and_returns_a_status(ops):
    """A wait on a peer's arrival counter that nothing will ever advance must give up at its deadline, leave
    TIMEOUT_FLAG in the status block and return normally: the context stays usable afterwards."""
    from skygdr_b200._ext import load

    C = load()
    rows, hidden = 4, 1024
    resid = torch.randn((rows, hidden), dtype=torch.bfloat16, device="cuda")
    w = torch.ones(hidden, dtype=torch.bfloat16, device="cuda")
    rs_buf = torch.zeros((1, rows, hidden), dtype=torch.bfloat16, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")          # stays 0: the "peer" never arrives
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    ag = torch.zeros((rows, hidden), dtype=torch.bfloat16, device="cuda")
    ag_ctr = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = ops.new_status("cuda")
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    C.tp_norm(rs_buf.data_ptr(), counter.data_ptr(), (step.data_ptr(), 1, 0, 5), resid, w, [ag.data_ptr()], [ag_ctr.data_ptr()], 0, 1e-6,
              20_000_000, status)                                          # 20 ms deadline
    t1.record()
    torch.cuda.synchronize()
    st = ops.read_status(status)
    assert st["status_name"] == "TIMEOUT_FLAG" and 100 <= st["detail"] < 100 + rows
    assert 15.0 < t0.elapsed_time(t1) < 500.0
    assert int(ag_ctr.item()) == rows                                      # it still finished its own work and signalled
    # the context is alive: an ordinary kernel runs and gives the right answer
    x = torch.randn((8, 512), dtype=torch.bfloat16, device="cuda")
    y = ops.rmsnorm(x, torch.ones(512, dtype=torch.bfloat16, device="cuda"), 1e-6)
    xf = x.float()
    assert torch.allclose(y.float(), xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6), atol=2e-2, rtol=2e-2)
    # once a status is set, later waits of the same engine are skipped instead of each burning a deadline
    t0.record()
    C.tp_norm(rs_buf.data_ptr(), counter.data_ptr(), (step.data_ptr(), 1, 0, 5), resid, w, [ag.data_ptr()], [ag_ctr.data_ptr()], 0, 1e-6,
              20_000_000, status)
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 10.0


def test_gemm_tile_and_split_choices_agree_with_reference(ops):
    """Every (token tile, split) the cost model may choose gives the same product."""
    torch.manual_seed(9)
    M, N, K = 128, 768, 4096
    x = torch.randn((M, K), dtype=torch.bfloat16, device="cuda")
    w = (torch.randn((N, K), dtype=torch.bfloat16, device="cuda") / 64).contiguous()
    ref = x.float() @ w.float().t()
    for ntok, splits in [(16, 1), (32, 5), (64, 2), (128, 1), (128, 3), (32, 1)]:
        y = ops.gemm(x, w, splits=splits, ntok=ntok)
        assert (y.float() - ref).abs().max() < 2e-2 * float(ref.abs().max()), (ntok, splits)
    nt, sp = ops.pick_config(M, N, K, 148)
    assert nt in (16, 32, 64, 128) and 1 <= sp <= 16


def test_cli_programs_run(ops):
    """The command-line programs print the reference's summary lines."""
    import re
    import subprocess
    import sys

    def run(mod, *args):
        r = subprocess.run([sys.executable, "-m", f"skygdr_b200.cli.{mod}", *args], capture_output=True, text=True, timeout=180)
        assert r.returncode == 0, r.stdout + r.stderr
        return r.stdout

    out = run("gpu_memhog", "--gb=1", "--op=copy", "--seconds=0", "--iters=3")
    assert re.search(r"\[memhog\] bytes=\d+ kernel_s=[0-9.]+ bw_gib_s=[0-9.]+", out)
    out = run("decode_hbm_stress", "0", "1024", "5")
    assert re.search(r"HBM stress done: approx [0-9.]+ GiB in [0-9.]+ s = [0-9.]+ GiB/s", out)
    assert re.search(r"gpu=0 name=.+ working_set=1024 MiB iters=5", out)
    out = run("gpu_pcie_memcpy", "--seconds=0", "--total_bytes=256M", "--chunk_mb=16", "--streams=2", "--batch=1", "--inflight=2", "--dir=h2d",
              "--report_ms=50")
    assert "[pcie] t=" in out and re.search(r"\[pcie\] done dir=h2d completed_bytes=268435456", out)
    out = run("kv_nvlink_transfer", "0", "0", "256", "3", "--layers", "4")
    assert re.search(r"KV transfer done: [0-9.]+ GiB in [0-9.]+ s = [0-9.]+ GiB/s", out) and "src_gpu=0 dst_gpu=0 size=256 MiB iters=3" in out
    out = run("kv_nvlink_transfer_trace", "--src", "0", "--dst", "0", "--iters", "5", "--dist", "computed", "--layers", "4", "--max-tokens", "4096")
    assert "Trace-shaped KV transfer done:" in out and "transfers: 5" in out
    for label in ("src_gpu=0 dst_gpu=0 iters=5 dist=computed", "KV geometry: layers=4 kv_heads=8 head_dim=128 elem_bytes=2", "Trace quantiles: p50=758",
                  "sampled tokens: p50=", "sampled bytes: p50=", "max transfer allocation:"):
        assert label in out, label
    out = run("decode_kvcache_stress", "--layers", "2", "--context", "2048", "--gen", "4", "--batch", "4")
    assert "Effective sequence-throughput:" in out and "Approx bandwidth:" in out


@pytest.mark.parametrize("M,N,K,gated,ntok", [(2048, 1024, 1024, False, 0), (300, 640, 512, False, 0), (1000, 200, 256, False, 128),
                                              (777, 384, 1024, True, 0), (40000, 256, 128, False, 0)])
def test_persistent_gemm_matches_reference(ops, M, N, K, gated, ntok):
    """One CTA per SM walking the output tiles with two TMEM accumulators: full tiles, ragged tokens and features, a gated
    case, and a case with far more tiles than CTAs (every accumulator and every ring slot is reused many times)."""
    from skygdr_b200.ops.gemm import workspace_for

    torch.manual_seed(12)
    x = torch.randn((M, K), dtype=torch.bfloat16, device="cuda")
    w = (torch.randn((N * (2 if gated else 1), K), dtype=torch.bfloat16, device="cuda") / math.sqrt(K)).contiguous()
    y = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm(x, w, out=y, gated=gated, ntok=ntok, persistent=True)
    ref = x.float() @ w.float().t()
    if gated:
        ref = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:]
    torch.cuda.synchronize()
    assert ops.read_status(workspace_for("cuda").status)["status"] == 0
    err = (y.float() - ref).abs().max()
    assert err < 2e-2 * max(1.0, float(ref.abs().max())), float(err)
    y2 = ops.gemm(x, w, gated=gated)                      # the one-tile-per-CTA kernel must agree to rounding
    assert (y.float() - y2.float()).abs().max() < 2e-2 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("M,N,K,gated", [(2048, 1024, 1024, False), (300, 512, 512, False), (1000, 256, 256, False), (40000, 256, 128, False),
                                         (2048, 1024, 1024, True), (777, 384, 1024, True), (300, 200, 512, True), (40000, 128, 128, True)])
def test_persistent_gemm_with_wide_tiles_matches_reference(ops, M, N, K, gated):
    """Two weight blocks per 256-token operand (both accumulators of TMEM in one tile, two epilogue groups): 256 x 256 tiles, or a
    gate and an up block for 128 gated outputs; full tiles, ragged tokens and features, and far more tiles than CTAs
    (accumulators and ring slots reused many times)."""
    from skygdr_b200.ops.gemm import workspace_for

    torch.manual_seed(13)
    x = torch.randn((M, K), dtype=torch.bfloat16, device="cuda")
    w = (torch.randn((N * (2 if gated else 1), K), dtype=torch.bfloat16, device="cuda") / math.sqrt(K)).contiguous()
    y = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm(x, w, out=y, gated=gated, persistent="wide")
    ref = x.float() @ w.float().t()
    if gated:
        ref = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:]
    torch.cuda.synchronize()
    assert ops.read_status(workspace_for("cuda").status)["status"] == 0
    err = (y.float() - ref).abs().max()
    assert err < 2e-2 * max(1.0, float(ref.abs().max())), float(err)
    y2 = ops.gemm(x, w, gated=gated, persistent="narrow")
    assert (y.float() - y2.float()).abs().max() < 2e-2 * max(1.0, float(ref.abs().max()))


def test_temperature_sampling_matches_the_cpu_restatement(ops):
    """Gumbel-max sampling: the kernel's pick must be the CPU oracle's pick (same hash, fp32 arithmetic), except where the two
    best perturbed values are within rounding of each other; positions change the draw, the seed changes the stream."""
    torch.manual_seed(21)
    rows, vocab = 48, 151936
    logits = (torch.randn((rows, vocab), device="cuda") * 2.0).to(torch.bfloat16)
    pos = torch.randint(0, 30000, (rows,), dtype=torch.int32, device="cuda")
    got = ops.sample(logits, 0.7, seed=99, positions=pos).cpu()
    want, v = ops.sample_reference(logits.cpu(), 0.7, 99, pos.cpu())
    picked = v.gather(1, got.long()[:, None])[:, 0]
    assert bool((picked >= v.max(-1).values - 1e-3).all())                 # the maximum, up to the accuracy of the fast logarithm
    assert float((got == want).float().mean()) > 0.9
    assert torch.equal(ops.sample(logits, 0.7, seed=99, positions=pos).cpu(), got)         # deterministic
    assert not torch.equal(ops.sample(logits, 0.7, seed=99, positions=pos + 1).cpu(), got)
    assert not torch.equal(ops.sample(logits, 0.7, seed=100, positions=pos).cpu(), got)
    greedy = ops.argmax(logits).cpu()
    assert float((ops.sample(logits, 1e-3, seed=1, positions=pos).cpu() == greedy).float().mean()) > 0.95


def test_kernel_is_paced_by_the_daemon_process_through_the_page_it_owns(ops):
    """The product's minimum slice on one GPU: a `fabricd` process owns the credit page (a file under /dev/shm), a flow registers
    over TCP, maps that page into the device's address space (CreditPage.attach) and launches the paged transfer kernel, which
    reads the daemon's grants chunk by chunk. Under the `static` policy a best-effort flow gets half of its link's capacity:
    the kernel runs out of credit, yields, is relaunched from its cursor, and ends up moving its bytes at the granted rate,
    bit-exact. Unpaced (policy none), the same transfer is many times faster."""
    import struct
    import time

    from skygdr_b200.control import FabricClient, FabricDaemon

    geom = ops.KVGeometry(layers=8, kv_heads=8)
    nb = 256                                                   # 256 blocks x 512 KiB = 134 MB
    src = ops.PagedKVPool(geom, nb, "nhd")
    src.data.normal_()
    dst = ops.PagedKVPool(geom, nb, "hnd")
    g = torch.Generator().manual_seed(2)
    sb = torch.randperm(nb, generator=g).int().cuda()
    db = torch.randperm(nb, generator=g).int().cuda()
    total = ops.link_bytes(geom, nb)
    rates = {}
    for policy, cap in (("static", 8.0), ("none", 8.0)):       # static: LOW1 = half of the 8 GB/s link = 4 GB/s
        with FabricDaemon(policy=policy, window_us=1000, lease_ms=60000, extra=["--link", f"test={cap}"]) as d, FabricClient(port=d.port) as c:
            h = c.register("kv_bulk", 0, 0.0, kind="kv_offload", link="test")
            assert h.page_path and h.page_path.startswith("/dev/shm/")
            page = ops.CreditPage.attach(h.page_path)
            try:
                struct.pack_into("<Q", h._mm, 128 + 56, total)          # backlog: the flow has this much to send
                flow = ops.KvTransferFlow("cuda", page=page, max_wait_ms=2.0)
                dst.data.zero_()
                t0 = time.perf_counter()
                st = flow.transfer_to_completion(src, [ops.RemotePool.of(dst)], sb, db)
                dt = time.perf_counter() - t0
                # a launch that ran out of credit is resumed from the lowest unfinished chunk: chunks past it that other CTAs had
                # already moved are moved again, so the byte count may exceed the payload by a few chunks
                assert st["status"] == 0 and total <= st["bytes_done"] <= total * 1.1, st
                assert torch.equal(dst.data[db.long()], ops.reference_transfer(src, sb))
                rates[policy] = (total / dt / 1e9, st["launches"])
                usage = h.usage()
                assert usage["completed_bytes"] >= total                # the kernel wrote its progress into the daemon's page
                if policy == "static":
                    assert h.grant()["unlimited"] == 0 and h.grant()["granted_bytes"] >= total
            finally:
                page.close()
                c.unregister(h)
    paced, launches = rates["static"]
    assert 2.5 < paced < 5.0, rates                            # 4 GB/s granted; start-up and relaunch gaps cost a little
    assert launches > 3, rates                                 # it yielded and resumed
    assert rates["none"][0] > 10 * paced, rates
