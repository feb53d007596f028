"""The entry point for callers that may not allocate device memory
(kvcore_b200/csrc/no_alloc_api.h): some hosts hand every library a fixed share of the GPU and
forbid cudaMalloc inside it, others sit on a path where the allocator's device-wide
synchronisation is not acceptable.  For them the split-KV attention keeps its scratch in an
array built into the library.  This test calls that entry point through its exported C symbol,
twice in a row on different inputs (the second call finds the first call's leftovers in the
shared array; one pair is ordered so that the second call has more requests and more splits than
the first and therefore reads rows of the array the first never wrote), and checks each result
against the regular entry point, which takes caller scratch, and against the plain statement of
paged attention in tests/plain_kernels.py.  It also checks that a request larger than the built-in
array is refused, and that a problem one call reports is still on record after a later, clean call.

Collected last on purpose: a run that stops at the first failure has then run everything else.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
STATIC_SCRATCH_FLOATS = 2 * 1024 * 1024


def _library():
    import kvcore_b200.kernels as K

    K.require_device(DEV)
    lib = ctypes.CDLL(K.ensure_built())
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.kvb_flash_paged_attention_static.argtypes = [vp, i64, vp, i64, vp, vp, vp, i32, vp, vp, i32, i32, i32,
                                                     i32, i32, i32, i32, f32, i32, i32, vp]
    lib.kvb_flash_paged_attention_static.restype = i32
    lib.kvb_static_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    lib.kvb_static_status.restype = i32
    lib.kvb_last_error.restype = ctypes.c_char_p
    return K, lib


def _case(seed, heads, kv_heads, dim, page, lens):
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-(c + q) // page) for c, q in lens]
    total = sum(pages_per) + 1
    perm = (torch.randperm(total - 1, generator=g) + 1).to(torch.int32)
    table = torch.zeros((len(lens), max(pages_per)), dtype=torch.int32)
    cursor = 0
    for r, n in enumerate(pages_per):
        table[r, :n] = perm[cursor:cursor + n]
        cursor += n
    k = (torch.randn(total, kv_heads, page, dim, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    v = (torch.randn(total, kv_heads, page, dim, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    tokens = sum(q for _, q in lens)
    qkv = torch.randn(tokens, (heads + 2 * kv_heads) * dim, generator=g).to(torch.bfloat16).to(DEV)
    starts = [0]
    for _, q in lens:
        starts.append(starts[-1] + q)

    class Ctx:
        pass

    ctx = Ctx()
    ctx.num_reqs = len(lens)
    ctx.max_query_len = max(q for _, q in lens)
    ctx.max_seq_len = max(c + q for c, q in lens)
    ctx.query_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    ctx.context_lens = torch.tensor([c for c, _ in lens], dtype=torch.int32, device=DEV)
    ctx.positions = torch.cat([torch.arange(c, c + q, dtype=torch.int32) for c, q in lens]).to(DEV)
    ctx.req_index = torch.cat([torch.full((q,), r, dtype=torch.int32) for r, (_, q) in enumerate(lens)]).to(DEV)
    return qkv, k, v, table.to(DEV), ctx


def _call_static(lib, qkv, k, v, table, ctx, heads, kv_heads, dim, scale, window, splits):
    out = torch.full((qkv.shape[0], heads * dim), float("nan"), dtype=torch.bfloat16, device=DEV)
    num_pages, _, page, _ = k.shape
    code = lib.kvb_flash_paged_attention_static(
        out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0), k.data_ptr(), v.data_ptr(),
        table.data_ptr(), table.stride(0), ctx.query_start.data_ptr(), ctx.context_lens.data_ptr(),
        ctx.num_reqs, ctx.max_query_len, heads, kv_heads, dim, page, num_pages, scale, window, splits,
        torch.cuda.current_stream().cuda_stream)
    return code, out


def test_static_scratch_entry_point_matches_the_regular_one_and_the_plain_statement():
    import plain_kernels

    K, lib = _library()
    shapes = [
        (10, 8, 2, 128, 16, [(260, 1), (40, 1)], 0, 2),              # small: few rows of the array written
        (11, 32, 8, 128, 16, [(700, 1), (17, 1), (1500, 1), (0, 1), (333, 1)], 0, 7),   # more requests, heads and
                                                                     # splits: reads rows the call before never wrote
        (12, 8, 2, 64, 8, [(300, 2), (64, 1), (900, 3)], 0, 5),      # other sizes: leftovers of call two lie underneath
        (13, 8, 2, 128, 16, [(900, 1), (70, 1)], 100, 4),            # window
        (14, 6, 2, 96, 16, [(5, 150), (0, 3)], 0, 1),                # one split, tile shape: no scratch used
    ]
    for seed, heads, kv_heads, dim, page, lens, window, splits in shapes:
        qkv, k, v, table, ctx = _case(seed, heads, kv_heads, dim, page, lens)
        scale = dim ** -0.5
        want = K.paged_attention(qkv, k, v, table, ctx, heads, kv_heads, dim, scale, window or None,
                                 num_splits=splits, use_tma=False)
        plain = plain_kernels.paged_attention_plain(qkv.float(), k.float(), v.float(), table, ctx.positions,
                                                    ctx.req_index, heads, kv_heads, dim, scale, window or None)
        for _ in range(2):  # two calls in a row
            code, got = _call_static(lib, qkv, k, v, table, ctx, heads, kv_heads, dim, scale, window, splits)
            assert code == 0, lib.kvb_last_error().decode()
            torch.cuda.synchronize()
            assert torch.isfinite(got.float()).all()
            torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
            torch.testing.assert_close(got.float(), plain, rtol=2e-2, atol=2e-2)
        status = ctypes.c_int(-1)
        assert lib.kvb_static_status(ctypes.byref(status)) == 0 and status.value == 0


def test_a_reported_problem_outlives_the_calls_behind_it():
    """A page id outside the cache is not read: the kernel skips it and sets a status bit.  The bit is
    still there after a later call that had nothing to report, and is cleared by reading it."""
    K, lib = _library()
    heads, kv_heads, dim, page = 8, 2, 128, 16
    qkv, k, v, table, ctx = _case(21, heads, kv_heads, dim, page, [(200, 1), (90, 1)])
    broken = table.clone()
    broken[0, 3] = k.shape[0] + 5
    code, _ = _call_static(lib, qkv, k, v, broken, ctx, heads, kv_heads, dim, dim ** -0.5, 0, 3)
    assert code == 0
    code, got = _call_static(lib, qkv, k, v, table, ctx, heads, kv_heads, dim, dim ** -0.5, 0, 3)
    assert code == 0
    status = ctypes.c_int(-1)
    assert lib.kvb_static_status(ctypes.byref(status)) == 0 and status.value == 2
    assert lib.kvb_static_status(ctypes.byref(status)) == 0 and status.value == 0
    assert torch.isfinite(got.float()).all()
    code, _ = _call_static(lib, qkv, k, v, table, ctx, heads, kv_heads, dim, dim ** -0.5, 0, 5000)
    assert code != 0 and "at most 1024 splits" in lib.kvb_last_error().decode()


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    K, lib = _library()
    heads, kv_heads, dim, page = 32, 8, 128, 16
    lens = [(40, 1)] * 64
    qkv, k, v, table, ctx = _case(15, heads, kv_heads, dim, page, lens)
    splits = 4
    assert 64 * kv_heads * splits * 16 * (dim + 2) > STATIC_SCRATCH_FLOATS
    code, _ = _call_static(lib, qkv, k, v, table, ctx, heads, kv_heads, dim, dim ** -0.5, 0, splits)
    assert code != 0
    assert "exceeds the built-in scratch" in lib.kvb_last_error().decode()
    code, got = _call_static(lib, qkv, k, v, table, ctx, heads, kv_heads, dim, dim ** -0.5, 0, 1)
    assert code == 0  # without splits nothing is needed
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()
