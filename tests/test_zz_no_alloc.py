"""The allocation-free C entry point for paged decode attention (its scratch is a fixed array inside the
library) must agree with the regular entry point, which takes torch-allocated scratch.

Callers of that entry point are programs that cannot allocate device memory when they need attention
(all HBM already handed to another allocator, no tolerance for the implicit synchronisation of
cudaMalloc, or a C plug-in with no tensor library). This test plays such a caller: it finds the exported
symbol with ctypes, passes raw device pointers, and never hands it any scratch. Two calls in a row with
different inputs check that what the first call leaves in the shared scratch does not leak into the second.
The file name sorts last so that a run that stops at the first failure has run everything else before.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from skygdr_b200 import build
    from skygdr_b200._ext import load

    load()  # builds if needed and pulls in the CUDA runtime and torch libraries the .so depends on
    lib = ctypes.CDLL(str(build.cuda_path()))
    fn = lib.skygdr_paged_attn_decode_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong,
                   ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    # the start-up call such a caller makes once per device, before its memory is handed away and before any capture
    init = lib.skygdr_paged_attn_noalloc_init
    init.restype = ctypes.c_int
    init.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    err = ctypes.create_string_buffer(256)
    assert init(err, 256) == 0, err.value.decode()
    assert init(err, 256) == 0                       # idempotent
    fn.read_status = lib.skygdr_paged_attn_noalloc_status
    fn.read_status.restype = ctypes.c_int
    fn.read_status.argtypes = [ctypes.POINTER(ctypes.c_uint), ctypes.POINTER(ctypes.c_uint), ctypes.c_void_p]
    return fn


def _kernel_status(fn):
    code, detail = ctypes.c_uint(99), ctypes.c_uint(0)
    assert fn.read_status(ctypes.byref(code), ctypes.byref(detail), torch.cuda.current_stream().cuda_stream) == 0
    return code.value, detail.value


def _case(ops, seed, ctx_list, kv_heads=8, q_heads=32):
    torch.manual_seed(seed)
    g = ops.KVGeometry(layers=2, kv_heads=kv_heads)
    ctx = torch.tensor(ctx_list, dtype=torch.int32, device="cuda")
    B = ctx.numel()
    max_blocks = (int(ctx.max()) + 15) // 16
    nblk = int(((ctx + 15) // 16).sum()) + 3
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
    return g, pool, table, ctx, q


def _call(fn, pool, layer, table, ctx, q, kv_heads, chunk, max_ctx=None):
    out = torch.zeros_like(q)
    bs, ls, ks = pool.strides
    err = ctypes.create_string_buffer(512)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(q.data_ptr(), pool.layer_base(layer).data_ptr(), out.data_ptr(), table.data_ptr(), ctx.data_ptr(), bs, ks,
            pool.head_stride, q.shape[0], q.shape[1], kv_heads, table.shape[1], pool.data.shape[0], max_ctx or int(ctx.max()), chunk,
            1.0 / 128 ** 0.5, stream, err, 512)
    return rc, out, err.value.decode()


def test_no_alloc_entry_matches_regular_entry_twice():
    import skygdr_b200.ops as ops

    fn = _entry()
    for seed, ctx_list, layer in ((11, [700, 1, 64, 2049, 513, 16], 0), (12, [33, 1500, 1024, 5], 1)):
        g, pool, table, ctx, q = _case(ops, seed, ctx_list)
        rc, got, msg = _call(fn, pool, layer, table, ctx, q, 8, 512)
        assert rc == 0, msg
        assert _kernel_status(fn) == (0, 0)          # the kernel ran to the end and met nothing to report
        attn = ops.PagedAttention("cuda", q.shape[0], 32, 8, max_ctx=4096, chunk_tokens=512)
        want = attn(q, pool, layer, table, ctx, max_ctx=int(ctx.max()))
        torch.cuda.synchronize()
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), float((got.float() - want.float()).abs().max())
        ref = ops.paged_attn_reference(q, pool, layer, table, ctx)
        assert torch.allclose(got.float(), ref, atol=2e-2, rtol=2e-2)


def test_no_alloc_entry_rejects_oversize_and_bad_arguments():
    import skygdr_b200.ops as ops

    fn = _entry()
    g, pool, table, ctx, q = _case(ops, 13, [100, 200])
    bs, ls, ks = pool.strides
    err = ctypes.create_string_buffer(512)
    args = [q.data_ptr(), pool.layer_base(0).data_ptr(), q.data_ptr(), table.data_ptr(), ctx.data_ptr(), bs, ks, pool.head_stride]
    # 4096 sequences x 32 heads x 1 split = 131072 rows: beyond the built-in scratch
    nb = pool.data.shape[0]
    rc = fn(*args, 4096, 32, 8, table.shape[1], nb, 200, 512, 0.1, None, err, 512)
    assert rc == -1 and b"exceeds the built-in scratch" in err.value
    rc = fn(*args, 2, 32, 8, table.shape[1], nb, 200, 100, 0.1, None, err, 512)
    assert rc == -2 and b"multiple of 64" in err.value
    rc = fn(None, *args[1:], 2, 32, 8, table.shape[1], nb, 200, 512, 0.1, None, err, 512)
    assert rc == -2
    # unsupported geometry is refused before anything is enqueued: 24 query heads on 8 KV heads (group of 3), and a
    # max_ctx that the block-table row cannot cover
    rc = fn(*args, 2, 24, 8, table.shape[1], nb, 200, 512, 0.1, None, err, 512)
    assert rc == -2 and b"1, 2, 4 or 8" in err.value
    rc = fn(*args, 2, 32, 8, table.shape[1], nb, table.shape[1] * 16 + 1, 512, 0.1, None, err, 512)
    assert rc == -2 and b"covers only" in err.value


def test_no_alloc_entry_reports_bad_lengths_and_block_ids_without_touching_them():
    """Stale device data from the caller (a context length beyond max_ctx, a block id outside the pool) must come back as a
    status word, not as a read outside the pool: the length is cut to max_ctx, the block id is replaced by block 0, and the
    sequences that were not affected still get their exact result."""
    import skygdr_b200.ops as ops

    fn = _entry()
    g, pool, table, ctx, q = _case(ops, 14, [300, 520, 77])
    ref = ops.paged_attn_reference(q, pool, 0, table, ctx)
    # (a) sequence 1 claims more tokens than max_ctx says any sequence has
    bad_ctx = ctx.clone()
    bad_ctx[1] = 5000
    rc, got, msg = _call(fn, pool, 0, table, bad_ctx, q, 8, 256, max_ctx=520)
    assert rc == 0, msg
    code, detail = _kernel_status(fn)
    assert code == 4 and detail == (0x40000000 | 1), (code, hex(detail))
    assert torch.allclose(got.float(), ref, atol=2e-2, rtol=2e-2)          # cut to 520 = its true length: still the right answer
    # (b) one table entry of sequence 0 names a block far outside the pool
    bad_table = table.clone()
    bad_table[0, 3] = 10 ** 6
    rc, got, msg = _call(fn, pool, 0, bad_table, ctx, q, 8, 256)
    assert rc == 0, msg
    code, detail = _kernel_status(fn)
    assert code == 4 and detail == ((0 << 16) | 3), (code, hex(detail))
    assert torch.allclose(got[1:].float(), ref[1:], atol=2e-2, rtol=2e-2)  # the other sequences are untouched
    # and a clean call afterwards starts from a clean status
    rc, got, msg = _call(fn, pool, 0, table, ctx, q, 8, 256)
    assert rc == 0 and _kernel_status(fn) == (0, 0)
    assert torch.allclose(got.float(), ref, atol=2e-2, rtol=2e-2)
