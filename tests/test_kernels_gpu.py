"""Each CUDA kernel alone against its plain PyTorch statement (tests/plain_kernels.py), in
float32 and bfloat16, at sizes other than the engine's tiny models: widths that are no
power of two, head sizes in steps of 16, odd head counts and groups, pages that are not
full, windows."""
from __future__ import annotations

import pytest
import torch

import plain_kernels as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def K():
    import kvcore_b200.kernels as kernels

    kernels.require_device(DEV)
    return kernels


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-3)


def randn(*shape, dtype, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,count", [(301, 120, 17), (1000, 4096, 64), (37, 7, 5)])
def test_gather_rows(dtype, rows, width, count):
    table = randn(rows, width, dtype=dtype)
    ids = torch.randint(0, rows, (count,), dtype=torch.int32, device=DEV)
    out = K().gather_rows(table, ids)
    assert torch.equal(out, P.gather_rows(table, ids))
    assert K().read_status() == 0


def test_feed_tokens():
    ids = torch.arange(100, 137, dtype=torch.int32, device=DEV)
    source = torch.full((37,), -1, dtype=torch.int32, device=DEV)
    source[[0, 5, 36]] = torch.tensor([2, 0, 2], dtype=torch.int32, device=DEV)
    sampled = torch.tensor([7, 8, 9], dtype=torch.int32, device=DEV)
    want = ids.clone()
    P.feed_tokens(want, source, sampled)
    K().feed_tokens(ids, source, sampled)
    assert torch.equal(ids, want) and ids[0] == 9 and ids[5] == 7 and ids[36] == 9 and ids[1] == 101
    assert K().read_status() == 0
    source[3] = 3                                # a row the sampler output does not have: flagged, not read
    K().feed_tokens(ids, source, sampled)
    assert ids[3] == 103 and K().read_status() & 1


def test_gather_rows_flags_bad_id():
    table = randn(10, 8, dtype=torch.float32)
    ids = torch.tensor([3, 10, -1], dtype=torch.int32, device=DEV)
    out = K().gather_rows(table, ids)
    assert torch.equal(out[0], table[3]) and not out[1:].any()
    assert K().read_status() & 1
    assert K().read_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(5, 96), (33, 4096), (3, 1001), (2, 8192 + 8)])
def test_rmsnorm(dtype, rows, width):
    x = randn(rows, width, dtype=dtype, seed=1)
    w = randn(width, dtype=dtype, seed=2)
    torch.testing.assert_close(K().rmsnorm(x, w, 1e-5), P.rmsnorm(x, w, 1e-5), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(5, 96), (33, 4096), (3, 1001)])
def test_add_rmsnorm(dtype, rows, width):
    h = randn(rows, width, dtype=dtype, seed=1)
    res = randn(rows, width, dtype=dtype, seed=3)
    w = randn(width, dtype=dtype, seed=2)
    res_ref = res.clone()
    want = P.add_rmsnorm(h, res_ref, w, 1e-6)
    got = K().add_rmsnorm(h, res, w, 1e-6)
    assert torch.equal(res, res_ref)  # the sum is a single correctly rounded addition
    torch.testing.assert_close(got, want, **tol(dtype))


def test_rmsnorm_keeps_32bit_weight_in_bf16_model():
    x = randn(7, 200, dtype=torch.bfloat16, seed=1)
    w = randn(200, dtype=torch.float32, seed=2)
    want = (w * (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5))).to(torch.bfloat16)
    torch.testing.assert_close(K().rmsnorm(x, w, 1e-5), want, **tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter", [(9, 160), (64, 14336), (3, 37)])
def test_silu_mul(dtype, rows, inter):
    gu = randn(rows, 2 * inter, dtype=dtype, seed=4)
    torch.testing.assert_close(K().silu_mul(gu), P.silu_mul(gu), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter,group", [(9, 160, 8), (64, 14336, 8), (3, 36, 4), (5, 30, 3)])
def test_silu_mul_with_alternating_runs(dtype, rows, inter, group):
    gu = randn(rows, 2 * inter, dtype=dtype, seed=4)
    got = K().silu_mul(gu, group)
    torch.testing.assert_close(got, P.silu_mul(gu, group), **tol(dtype))
    # the same numbers as the halves layout holds them
    runs = gu.view(rows, inter // group, 2, group)
    halves = torch.cat((runs[:, :, 0].reshape(rows, inter), runs[:, :, 1].reshape(rows, inter)), dim=1).contiguous()
    assert torch.equal(got, K().silu_mul(halves))


@pytest.mark.parametrize("m,n,k", [(1, 7, 5), (13, 200, 96), (70, 130, 257), (64, 64, 16), (3, 515, 96)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_f32(m, n, k, bias):
    x = randn(m, k, dtype=torch.float32, seed=5)
    w = randn(n, k, dtype=torch.float32, seed=6)
    b = randn(n, dtype=torch.float32, seed=7) if bias else None
    want = x.double() @ w.double().T + (b.double() if bias else 0)
    got = K().linear(x, w, b)
    torch.testing.assert_close(got.double(), want, rtol=1e-5, atol=1e-5)


def test_gemm_f32_rows_do_not_depend_on_batch():
    """A row's product is bit-identical whether it is computed alone or inside a larger batch."""
    x = randn(150, 300, dtype=torch.float32, seed=8)
    w = randn(130, 300, dtype=torch.float32, seed=9)
    full = K().linear(x, w)
    for rows in ([0], [149], [3, 77], list(range(64, 129))):
        part = K().linear(x[rows].contiguous(), w)
        assert torch.equal(part, full[rows])


@pytest.mark.parametrize("m,n,k", [(5, 96, 64), (77, 515, 96)])
def test_linear_bf16_and_32bit_logits(m, n, k):
    x = randn(m, k, dtype=torch.bfloat16, seed=5)
    w = randn(n, k, dtype=torch.bfloat16, seed=6, scale=0.1)
    want = x.float() @ w.float().T
    torch.testing.assert_close(K().linear(x, w).float(), want, rtol=2e-2, atol=2e-2)
    logits = K().linear(x, w, out_dtype=torch.float32)
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits, want, rtol=1e-3, atol=1e-3)


def _cache_case(dtype, heads, kv_heads, dim, page_size, lens, seed=0, window=None):
    """A batch of requests with contexts already in the cache plus new query tokens."""
    g = torch.Generator().manual_seed(seed)
    num_reqs = len(lens)
    total_pages = sum(-(-(c + q) // page_size) for c, q in lens) + 1
    perm = (torch.randperm(total_pages - 1, generator=g) + 1).tolist()  # scattered page ids
    width = max(-(-(c + q) // page_size) for c, q in lens)
    table = torch.zeros((num_reqs, width), dtype=torch.int32)
    cursor = 0
    for r, (c, q) in enumerate(lens):
        n = -(-(c + q) // page_size)
        table[r, :n] = torch.tensor(perm[cursor : cursor + n], dtype=torch.int32)
        cursor += n
    k_cache = randn(total_pages, kv_heads, page_size, dim, dtype=dtype, seed=seed + 1)
    v_cache = randn(total_pages, kv_heads, page_size, dim, dtype=dtype, seed=seed + 2)
    positions, req_index = [], []
    for r, (c, q) in enumerate(lens):
        positions += list(range(c, c + q))
        req_index += [r] * q
    tokens = len(positions)
    qkv = randn(tokens, (heads + 2 * kv_heads) * dim, dtype=dtype, seed=seed + 3)
    starts = [0]
    for _, q in lens:
        starts.append(starts[-1] + q)
    return dict(
        qkv=qkv, table=table.to(DEV), k_cache=k_cache, v_cache=v_cache,
        positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
        req_index=torch.tensor(req_index, dtype=torch.int32, device=DEV),
        query_start=torch.tensor(starts, dtype=torch.int32, device=DEV),
        context_lens=torch.tensor([c for c, _ in lens], dtype=torch.int32, device=DEV),
        lens=lens,
    )


class _Ctx:
    def __init__(self, case):
        self.positions, self.req_index = case["positions"], case["req_index"]
        self.query_start, self.context_lens = case["query_start"], case["context_lens"]
        self.num_reqs = len(case["lens"])
        self.max_query_len = max(q for _, q in case["lens"])
        self.max_seq_len = max(c + q for c, q in case["lens"])


ATTN_SHAPES = [
    # heads, kv_heads, dim, page, [(context, query), ...], window
    (4, 2, 16, 16, [(0, 7), (20, 1), (5, 13)], None),
    (3, 1, 32, 8, [(0, 40), (39, 1)], None),
    (6, 3, 48, 16, [(17, 30), (0, 1), (100, 2)], None),
    (5, 5, 80, 4, [(9, 9)], None),
    (8, 2, 128, 16, [(300, 1), (0, 64), (129, 3)], None),
    (4, 4, 256, 32, [(31, 34)], None),
    (4, 2, 64, 16, [(0, 50), (70, 1), (33, 5)], 24),
    (2, 1, 112, 16, [(40, 8)], 5),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,page,lens,window", ATTN_SHAPES)
def test_paged_attention(dtype, heads, kv_heads, dim, page, lens, window):
    case = _cache_case(dtype, heads, kv_heads, dim, page, lens)
    scale = dim ** -0.5
    got = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], _Ctx(case),
                              heads, kv_heads, dim, scale, window)
    want = P.paged_attention_plain(case["qkv"], case["k_cache"], case["v_cache"], case["table"],
                                   case["positions"], case["req_index"], heads, kv_heads, dim, scale, window)
    torch.testing.assert_close(got, want, **(dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32
                                             else dict(rtol=2e-2, atol=2e-2)))
    assert K().read_status() == 0


FLASH_SHAPES = [
    # heads, kv_heads, dim, page, [(context, query), ...], window, forced splits
    (32, 8, 128, 16, [(1000, 1), (17, 1), (4095, 1), (0, 1)], None, None),   # decode, split by the policy
    (32, 8, 128, 16, [(1000, 1), (17, 1), (300, 1)], None, 1),
    (32, 8, 128, 16, [(1000, 1), (17, 1), (300, 1)], None, 7),
    (32, 8, 128, 16, [(700, 4), (0, 2), (63, 3)], None, 3),                  # short portions ride the split kernel
    (8, 2, 64, 16, [(0, 200), (130, 77), (500, 1), (64, 64)], None, None),   # tiles, mixed with a decode
    (6, 2, 96, 8, [(5, 150), (0, 3)], None, None),                           # 3 heads a group: tokens straddle tiles
    (3, 1, 32, 8, [(0, 40), (39, 1)], None, None),
    (5, 5, 80, 4, [(9, 9), (100, 30)], None, None),
    (4, 4, 16, 32, [(31, 34), (0, 1)], None, None),
    (14, 2, 112, 16, [(40, 70)], None, None),
    (6, 3, 48, 16, [(17, 30), (0, 1), (100, 2)], None, None),
    (4, 2, 64, 16, [(0, 150), (170, 1), (33, 5)], 24, None),                 # window
    (8, 2, 128, 16, [(900, 1), (70, 1)], 100, 4),                            # window, decode, forced splits
    (8, 2, 128, 16, [(3000, 1), (1, 1), (640, 1)], None, 5),                 # TMA decode: ring wraps many times
    (16, 4, 64, 8, [(777, 1), (64, 2), (0, 1)], None, 3),                    # TMA decode: D=64, pages of 8
    (4, 1, 128, 64, [(500, 3), (63, 1)], None, 2),                           # TMA decode: pages of 64
    (2, 2, 64, 32, [(100, 9)], 17, None),                                    # TMA decode: 9 rows, window
    (8, 2, 128, 16, [(0, 200), (130, 77), (500, 1), (64, 64)], None, None),  # tcgen05 prefill, mixed with a decode
    (32, 8, 128, 16, [(0, 300)], None, None),                                # tcgen05 prefill: 3 key tiles, 10 row tiles
    (4, 1, 128, 64, [(1000, 130)], None, None),                              # tcgen05 prefill: long context, pages of 64
    (6, 2, 128, 8, [(5, 150), (0, 3)], None, None),                          # tcgen05 prefill: 3 heads a group
    (64, 8, 128, 16, [(1000, 1), (17, 1), (2047, 2), (0, 1)], None, None),   # TMA decode: 8 heads a group
    (16, 2, 128, 16, [(0, 200), (100, 50), (333, 1)], None, None),           # tcgen05 prefill: 8 heads a group
    (24, 8, 128, 16, [(1500, 1), (0, 1), (640, 1)], None, None),             # TMA decode: 3 heads a group
    # TMA decode with more (request, kv head, split) items than blocks that fit the GPU: blocks stay and share them
    (32, 8, 128, 16, [(37 * i % 700 + i % 3, 1) for i in range(50)], None, None),
    (32, 8, 128, 16, [(1000, 1), (17, 1), (4095, 1), (0, 1), (300, 2)], None, 13),   # with empty splits
    (16, 4, 64, 8, [(50 * i % 333, 1 + i % 2) for i in range(80)], None, None),
    (8, 2, 128, 32, [(0, 700)], 200, None),                                  # tcgen05 prefill: window
    (4, 4, 128, 16, [(250, 9), (0, 129)], None, None),                       # tcgen05 prefill: one head a group
]


@pytest.mark.parametrize("heads,kv_heads,dim,page,lens,window,splits", FLASH_SHAPES)
def test_flash_paged_attention(heads, kv_heads, dim, page, lens, window, splits):
    """The tensor-core kernel (tile and split shapes) against the plain statement and the general kernel."""
    dtype = torch.bfloat16
    case = _cache_case(dtype, heads, kv_heads, dim, page, lens, seed=7)
    # pages the batch does not own hold NaN: reading one shows up in the output (page 0 is the
    # null page, which the engine keeps zero: kernels that copy whole pages may read it)
    owned = set(case["table"].flatten().tolist()) | {0}
    case["k_cache"][0] = 0
    case["v_cache"][0] = 0
    for page_id in range(case["k_cache"].shape[0]):
        if page_id not in owned:
            case["k_cache"][page_id] = float("nan")
            case["v_cache"][page_id] = float("nan")
    # slots of owned pages beyond each request's length hold large stale values (finite, as
    # anything a kernel ever wrote to the cache is): they must not leak into the result
    for r, (c, q) in enumerate(lens):
        end = c + q
        last_page = int(case["table"][r, (end - 1) // page])
        if end % page:
            case["k_cache"][last_page, :, end % page:] = 3.0e4
            case["v_cache"][last_page, :, end % page:] = -3.0e4
    scale = dim ** -0.5
    ctx = _Ctx(case)
    assert K().flash_attention_supported(dtype, dim)
    got = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], ctx,
                              heads, kv_heads, dim, scale, window, num_splits=splits)
    no_tma = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], ctx,
                                 heads, kv_heads, dim, scale, window, num_splits=splits, use_tma=False,
                                 use_tc5=False)
    torch.testing.assert_close(got.float(), no_tma.float(), rtol=2e-2, atol=2e-2)
    general = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], ctx,
                                  heads, kv_heads, dim, scale, window, force_general=True)
    want = P.paged_attention_plain(case["qkv"], case["k_cache"], case["v_cache"], case["table"],
                                   case["positions"], case["req_index"], heads, kv_heads, dim, scale, window)
    assert torch.isfinite(got.float()).all()
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got.float(), general.float(), rtol=2e-2, atol=2e-2)
    assert K().read_status() == 0
    # the counters through which blocks share work are back at zero for the next launch
    assert all(not counters.any() for counters in K().api._decode_work_counters.values())


@pytest.mark.parametrize("seed", range(14))
def test_prompt_attention_on_tcgen05_random_batches(seed):
    """Batches drawn at random for the tcgen05 prompt kernel (head size 128): group sizes that divide 128
    (queries by TMA) and 3 (queries copied), every page size, windows, contexts that end anywhere in a key
    tile, portions that leave the second query tile of a block empty, partly filled, or one key tile behind
    the first.  Against the general kernel (itself checked against the plain statement), the first seeds
    against the plain statement as well."""
    import random

    rng = random.Random(1000 + seed)
    group = rng.choice([1, 2, 4, 8, 3, 4])
    kv_heads = rng.choice([1, 2])
    heads, dim = group * kv_heads, 128
    page = rng.choice([8, 16, 32, 64])
    window = rng.choice([None, None, rng.randint(20, 300)])
    lens = [(rng.choice([0, rng.randint(1, 700), 128 * rng.randint(0, 3), 127, 129]),
             rng.choice([rng.randint(17, 400), 32, 64, 65, 128 // group + 1]))
            for _ in range(rng.randint(1, 4))]
    lens[0] = (lens[0][0], max(lens[0][1], 16 // group + 1))         # at least one portion of more than 16 rows
    case = _cache_case(torch.bfloat16, heads, kv_heads, dim, page, lens, seed=seed)
    owned = set(case["table"].flatten().tolist()) | {0}
    case["k_cache"][0] = 0
    case["v_cache"][0] = 0
    for page_id in range(case["k_cache"].shape[0]):
        if page_id not in owned:
            case["k_cache"][page_id] = float("nan")
            case["v_cache"][page_id] = float("nan")
    scale = dim ** -0.5
    ctx = _Ctx(case)
    assert K().tc5_prefill_supported(torch.bfloat16, dim, page) and ctx.max_query_len * group > 16
    got = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], ctx,
                              heads, kv_heads, dim, scale, window)
    general = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], ctx,
                                  heads, kv_heads, dim, scale, window, force_general=True)
    assert torch.isfinite(got.float()).all(), (group, kv_heads, page, window, lens)
    torch.testing.assert_close(got.float(), general.float(), rtol=2e-2, atol=2e-2, msg=str((group, kv_heads, page, window, lens)))
    if seed < 3:
        want = P.paged_attention_plain(case["qkv"], case["k_cache"], case["v_cache"], case["table"],
                                       case["positions"], case["req_index"], heads, kv_heads, dim, scale, window)
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    assert K().read_status() == 0


MIXED_SHAPES = [
    # heads, kv_heads, dim, page, [(context, query), ...] longest portion first, window
    (32, 8, 128, 16, [(100, 300), (0, 64), (777, 1), (17, 1), (2047, 1), (0, 1)], None),   # tcgen05 + TMA decode
    (8, 2, 128, 16, [(5, 150), (900, 2), (64, 1), (33, 1)], None),                         # 2 tokens x 4 heads: still decode
    (6, 2, 128, 8, [(0, 70), (40, 9), (500, 5), (63, 1)], None),                           # 3 heads a group: 9 tokens are long
    (16, 4, 64, 8, [(10, 200), (300, 3), (77, 1)], None),                                  # mma.sync tile + TMA decode (D = 64)
    (6, 3, 48, 16, [(17, 130), (100, 2), (0, 1)], None),                                   # mma.sync tile + mma.sync split
    (8, 2, 128, 32, [(0, 400), (350, 1), (120, 1)], 100),                                  # window
]


@pytest.mark.parametrize("heads,kv_heads,dim,page,lens,window", MIXED_SHAPES)
def test_mixed_batches_go_to_two_kernels_and_give_one_result(heads, kv_heads, dim, page, lens, window):
    """A batch that says how long each request's portion is (longest first, as the step function packs
    it): portions of prompts and decoded tokens are handed to different kernels as two runs of requests,
    and every row is what the plain statement says (and what the one-kernel path gives)."""
    dtype = torch.bfloat16
    case = _cache_case(dtype, heads, kv_heads, dim, page, lens, seed=11)
    scale = dim ** -0.5
    ctx = _Ctx(case)
    one = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], ctx,
                              heads, kv_heads, dim, scale, window)
    launches = K().api.launch_count
    ctx.host_query_lens = [q for _, q in lens]
    ctx.host_context_lens = [c for c, _ in lens]
    two = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], ctx,
                              heads, kv_heads, dim, scale, window)
    assert K().api.launch_count - launches >= 2          # two kernels (and a merge where the decode run is split)
    want = P.paged_attention_plain(case["qkv"], case["k_cache"], case["v_cache"], case["table"],
                                   case["positions"], case["req_index"], heads, kv_heads, dim, scale, window)
    assert torch.isfinite(two.float()).all()
    torch.testing.assert_close(two.float(), want.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(two.float(), one.float(), rtol=2e-2, atol=2e-2)
    assert K().read_status() == 0


ROTATING_DECODE_SHAPES = [
    # heads, kv_heads, dim, page, [(context, query), ...], window, forced splits
    (32, 8, 128, 16, [(1000, 1), (17, 1), (4095, 1), (0, 1)], None, None),
    (32, 8, 128, 16, [(700, 4), (0, 2), (63, 3), (62, 4)], None, 3),      # new tokens straddle a tile and a split
    (16, 4, 64, 8, [(777, 1), (64, 2), (0, 1), (127, 1)], None, 3),
    (4, 1, 128, 64, [(500, 3), (63, 1), (191, 2)], None, 2),
    (2, 2, 64, 32, [(100, 9), (0, 16)], 17, None),                         # window; sixteen new tokens at once
    (6, 3, 48, 16, [(17, 2), (0, 1), (100, 2)], None, None),               # not the TMA kernel: kernel in front
    (64, 8, 128, 16, [(1000, 1), (0, 1), (63, 2)], None, None),            # 8 heads a group
    (24, 8, 128, 16, [(1500, 1), (0, 1), (640, 5)], None, 4),              # 3 heads a group, five new tokens
    (32, 8, 128, 16, [(29 * i % 500, 1 + i % 3) for i in range(40)], None, None),   # 320 items for 296 blocks
    (32, 8, 128, 16, [(61 * i % 900, 1) for i in range(14)], None, 3),             # 336 items, splits
    (8, 2, 128, 16, [(0, 200), (130, 77), (500, 1)], None, None),          # prefill shapes: kernel in front
]


@pytest.mark.parametrize("rotate", [True, False])
@pytest.mark.parametrize("heads,kv_heads,dim,page,lens,window,splits", ROTATING_DECODE_SHAPES)
def test_attention_that_rotates_and_writes_the_cache(heads, kv_heads, dim, page, lens, window, splits, rotate):
    """Rotation and cache write inside the attention call give the bits of the kernel in front."""
    dtype = torch.bfloat16
    case = _cache_case(dtype, heads, kv_heads, dim, page, lens, seed=11)
    ctx = _Ctx(case)
    tokens = case["qkv"].shape[0]
    cos_sin = None
    if rotate:
        angles = randn(tokens, dim // 2, dtype=torch.float32, seed=5) * 3.0
        cos_sin = torch.stack([angles.cos(), angles.sin()], dim=-1).contiguous()
    # the slots of this step's tokens hold large stale values before the step
    for r, (c, q) in enumerate(lens):
        for pos in range(c, c + q):
            page_id = int(case["table"][r, pos // page])
            case["k_cache"][page_id, :, pos % page] = 3.0e4
            case["v_cache"][page_id, :, pos % page] = -3.0e4
    scale = dim ** -0.5
    qkv_a, k_a, v_a = case["qkv"].clone(), case["k_cache"].clone(), case["v_cache"].clone()
    K().rope_kv_write(qkv_a, case["positions"], case["req_index"], cos_sin, case["table"], k_a, v_a,
                      heads, kv_heads, dim)
    want = K().paged_attention(qkv_a, k_a, v_a, case["table"], ctx, heads, kv_heads, dim, scale, window,
                               num_splits=splits)
    qkv_b, k_b, v_b = case["qkv"].clone(), case["k_cache"].clone(), case["v_cache"].clone()
    got = K().paged_attention(qkv_b, k_b, v_b, case["table"], ctx, heads, kv_heads, dim, scale, window,
                              num_splits=splits, cos_sin=cos_sin, write_kv=True)
    assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
    assert torch.equal(got, want)
    assert torch.isfinite(got.float()).all()
    # a layer that reads another layer's cache: the keys are there already, only q is rotated
    qkv_c = case["qkv"].clone()
    k_c, v_c = k_a.clone(), v_a.clone()
    borrowed = K().paged_attention(qkv_c, k_c, v_c, case["table"], ctx, heads, kv_heads, dim, scale, window,
                                   num_splits=splits, cos_sin=cos_sin, write_kv=False)
    assert torch.equal(borrowed, want)
    assert torch.equal(k_c, k_a) and torch.equal(v_c, v_a)
    assert K().read_status() == 0


def test_flash_split_policy():
    assert K().decode_splits(64, 8, 8192) == 1
    assert K().decode_splits(8, 8, 8192) == 7
    assert K().decode_splits(1, 8, 8192) == 32
    assert K().decode_splits(1, 8, 100) == 1
    assert K().decode_splits_tma(8, 8, 8192) == 4     # 256 blocks: one wave of 2 x 148
    assert K().decode_splits_tma(64, 8, 8192) == 1
    assert K().decode_splits_tma(1, 8, 8192) == 16
    assert K().decode_splits_tma(4, 8, 100) == 1
    assert K().decode_splits_tma(1, 8, 1024) == 8     # two tiles a split
    assert K().decode_splits_tma(8, 8, 1024) == 4
    assert K().decode_splits_tma(48, 8, 8192) == 2    # 1.3 waves unsplit: a sparse last wave
    assert K().decode_splits_tma(40, 8, 4096) == 4
    assert K().decode_splits_tma(37, 8, 8192) == 1    # exactly one wave
    assert K().tma_decode_supported(torch.bfloat16, 128, 16)
    assert not K().tma_decode_supported(torch.bfloat16, 96, 16)
    assert not K().tma_decode_supported(torch.float32, 128, 16)


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_finds_a_far_key(dtype):
    """One key among hundreds is made to dominate: the output must be that key's value."""
    heads, kv_heads, dim, page = 4, 2, 64, 16
    case = _cache_case(dtype, heads, kv_heads, dim, page, [(700, 1)], seed=3)
    far = 37  # position of the dominating key, on another page than the query
    q = case["qkv"][:, : heads * dim].view(1, heads, dim)
    page_id = int(case["table"][0, far // page])
    for head in range(heads):
        g = head // (heads // kv_heads)
        case["k_cache"][page_id, g, far % page] = (q[0, head].float() * 4.0).to(dtype)
    out = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], _Ctx(case),
                              heads, kv_heads, dim, 1.0, None).view(1, heads, dim)
    for head in range(heads):
        g = head // (heads // kv_heads)
        if head % (heads // kv_heads) == heads // kv_heads - 1:  # the head whose query the key copies last
            torch.testing.assert_close(out[0, head].float(), case["v_cache"][page_id, g, far % page].float(),
                                       rtol=2e-2, atol=2e-2)


WINDOW_EDGES = [
    # dtype, dim, page, (context, query), window, what runs
    (torch.float32, 64, 16, (300, 1), 100, dict(force_general=True)),
    (torch.bfloat16, 64, 16, (300, 1), 100, dict(force_general=True)),
    (torch.bfloat16, 128, 16, (300, 1), 100, dict(use_tma=False, use_tc5=False)),     # mma.sync, split shape
    (torch.bfloat16, 128, 16, (300, 1), 100, dict()),                                  # TMA decode
    (torch.bfloat16, 64, 8, (300, 1), 45, dict(num_splits=3)),                         # TMA decode: the edge on a tile's edge
    (torch.bfloat16, 128, 16, (170, 130), 100, dict(use_tma=False, use_tc5=False)),   # mma.sync, tile shape
    (torch.bfloat16, 128, 16, (170, 130), 100, dict()),                                # tcgen05 prefill
    (torch.bfloat16, 128, 32, (0, 400), 144, dict()),                                  # tcgen05 prefill: the edge on a tile's edge
]


@pytest.mark.parametrize("dtype,dim,page,lens,window,how", WINDOW_EDGES)
def test_paged_attention_at_the_windows_edge(dtype, dim, page, lens, window, how):
    """The last query row sees keys (pos - window, pos].  A key that dominates the row is put just
    inside that range: the output is its value.  Put just outside, with a huge value, it must leave no
    trace in the output."""
    heads = kv_heads = 2
    context, query = lens
    pos = context + query - 1
    for place, inside in ((pos - window + 1, True), (pos - window, False)):
        case = _cache_case(dtype, heads, kv_heads, dim, page, [lens], seed=13)
        q = case["qkv"][-1, : heads * dim].view(heads, dim)
        page_id = int(case["table"][0, place // page])
        for head in range(heads):
            case["k_cache"][page_id, head, place % page] = (q[head].float() * 4.0).to(dtype)
            if not inside:
                case["v_cache"][page_id, head, place % page] = 3.0e4
        out = K().paged_attention(case["qkv"], case["k_cache"], case["v_cache"], case["table"], _Ctx(case),
                                  heads, kv_heads, dim, 1.0, window, **how).view(query, heads, dim)[-1].float()
        assert K().read_status() == 0
        if inside:
            want = case["v_cache"][page_id, :, place % page].float()
            torch.testing.assert_close(out, want, rtol=2e-2, atol=2e-2)
        else:
            assert out.abs().max() < 10.0, "a key outside the window reached the output"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,page", [(4, 2, 16, 16), (3, 1, 32, 8), (6, 3, 48, 4), (32, 8, 128, 16)])
def test_rope_kv_write(dtype, heads, kv_heads, dim, page):
    lens = [(0, 9), (33, 1), (7, 12)]
    case = _cache_case(dtype, heads, kv_heads, dim, page, lens, seed=5)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))).float().to(DEV)
    ref = {k: v.clone() for k, v in case.items() if torch.is_tensor(v)}
    P.rope_kv_write(ref["qkv"], ref["positions"], ref["req_index"], P.rope_table(ref["positions"], inv_freq),
                    ref["table"], ref["k_cache"], ref["v_cache"], heads, kv_heads, dim)
    cos_sin = K().rope_table(case["positions"], inv_freq)
    torch.testing.assert_close(cos_sin, P.rope_table(case["positions"], inv_freq), rtol=1e-6, atol=1e-6)
    K().rope_kv_write(case["qkv"], case["positions"], case["req_index"], cos_sin, case["table"],
                      case["k_cache"], case["v_cache"], heads, kv_heads, dim)
    t = dict(rtol=1e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)
    torch.testing.assert_close(case["qkv"], ref["qkv"], **t)
    torch.testing.assert_close(case["k_cache"], ref["k_cache"], **t)
    assert torch.equal(case["v_cache"], ref["v_cache"])
    assert K().read_status() == 0


def test_rope_large_positions_fp32():
    """Angles of tens of thousands of radians keep full float accuracy."""
    dim, heads = 64, 2
    positions = torch.tensor([0, 1, 8191, 65535, 131071], dtype=torch.int32, device=DEV)
    q = randn(5, heads, dim, dtype=torch.float32, seed=1)
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))).float().to(DEV)
    want = P._rotate(q.cpu(), positions.cpu(), inv_freq.cpu())
    K().rope_inplace(q, None, positions, inv_freq)
    torch.testing.assert_close(q.cpu(), want, rtol=1e-5, atol=2e-6)


def test_kernels_refuse_cpu_tensors():
    import kvcore_b200.kernels as kernels

    with pytest.raises(kernels.KernelError, match="no CPU path"):
        kernels.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-5)
    with pytest.raises(kernels.KernelError):
        kernels.require_device("cpu")


# ---- sampling ---------------------------------------------------------------------------------
def _packed(rows):
    return torch.tensor(rows, dtype=torch.float64)


def test_sample_greedy_is_argmax_with_lowest_index():
    logits = randn(6, 515, dtype=torch.float32, seed=11)
    logits[2, 100] = logits[2, 400] = 50.0  # a tie: the lower index wins
    params = _packed([[0.0, 515, 1.0, 1, 0, 0]] * 6)
    got = K().sample(logits, params, 1e-5).cpu()
    want = logits.argmax(dim=-1).cpu()
    want[2] = 100
    assert got.tolist() == want.tolist()


def test_sample_matches_plain_noise_and_masks():
    vocab = 301
    logits = randn(8, vocab, dtype=torch.float32, seed=12, scale=2.0)
    rows = [
        [0.8, vocab, 1.0, 123, 0, 0],
        [0.8, vocab, 1.0, 123, 0, 1],
        [1.0, 5, 1.0, 7, 9, 3],
        [1.3, vocab, 0.7, 7, 9, 4],
        [0.5, 40, 0.9, 2**31 + 5, 2**31 + 1, 1000],
        [0.0, vocab, 1.0, 1, 1, 1],
        [2.0, 1, 1.0, 5, 5, 5],
        [1.0, vocab, 0.05, 5, 5, 6],
    ]
    got = K().sample(logits, _packed(rows), 1e-5).cpu().tolist()
    for row, (temperature, top_k, top_p, lo, hi, index) in enumerate(rows):
        seed = int(lo) | (int(hi) << 32)
        token, scores = P.sample_row(logits[row].cpu(), temperature, int(top_k), top_p, seed, int(index))
        if scores is None:
            assert got[row] == token
            continue
        assert torch.isfinite(scores[got[row]]), "sampled a masked token"
        # same token, or an exact near-tie of the noisy scores (rounding of exp/log differs)
        assert got[row] == token or abs(float(scores[got[row]] - scores[token])) < 1e-4
    assert got[0] != got[1] or True  # different token index -> different noise (may still coincide)


def test_sample_seeded_rows_do_not_depend_on_the_batch():
    vocab = 1000
    logits = randn(5, vocab, dtype=torch.float32, seed=13)
    rows = [[0.9, vocab, 1.0, 40 + r, 1, r] for r in range(5)]
    together = K().sample(logits, _packed(rows), 1e-5).cpu().tolist()
    alone = [K().sample(logits[r : r + 1].contiguous(), _packed([rows[r]]), 1e-5).item() for r in range(5)]
    assert together == alone
    again = K().sample(logits, _packed(rows), 1e-5).cpu().tolist()
    assert again == together


def test_sample_follows_the_distribution():
    vocab, draws = 16, 4000
    base = torch.linspace(-2.0, 2.0, vocab)
    logits = base.repeat(draws, 1).to(DEV).contiguous()
    rows = [[1.0, vocab, 1.0, 99, 0, i] for i in range(draws)]
    got = K().sample(logits, _packed(rows), 1e-5).cpu()
    counts = torch.bincount(got.long(), minlength=vocab).double()
    expected = torch.softmax(base.double(), dim=-1) * draws
    chi2 = float(((counts - expected) ** 2 / expected).sum())
    assert chi2 < 50.0, chi2  # 15 degrees of freedom: 50 is far in the tail


# ---- weight-streaming linear layer (decode) ---------------------------------------------------
@pytest.mark.parametrize("m,n,k", [
    (1, 64, 128), (3, 200, 64), (8, 4096, 4096), (8, 6144, 4096), (9, 515, 1024), (16, 130, 64),
    (13, 1024, 2048), (16, 96, 14336), (4, 4096, 1024), (5, 28672, 1024), (2, 70, 576),
    (8, 4096, 14336), (11, 4100, 1088), (7, 33, 3136),
])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_stream(m, n, k, bias):
    x = randn(m, k, dtype=torch.bfloat16, seed=20)
    w = randn(n, k, dtype=torch.bfloat16, seed=21, scale=0.05)
    b = randn(n, dtype=torch.bfloat16, seed=22) if bias else None
    want = x.float() @ w.float().T + (b.float() if bias else 0)
    got = K().linear_stream(x, w, b)
    assert got.dtype == torch.bfloat16
    torch.testing.assert_close(got.float(), want, rtol=1.6e-2, atol=2e-2)
    wide = K().linear_stream(x, w, b, out_dtype=torch.float32)
    torch.testing.assert_close(wide, want, rtol=1e-3, atol=2e-3)
    again = K().linear_stream(x, w, b, out_dtype=torch.float32)
    assert torch.equal(wide, again)  # halves and parts are added in a fixed order
    assert K().read_status() == 0


@pytest.mark.parametrize("m,inter,k", [(1, 64, 128), (8, 14336, 4096), (5, 200, 576), (16, 1000, 256), (3, 8, 64)])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_stream_with_gated_epilogue(m, inter, k, bias):
    """Rows in runs of 8 gate / 8 up: the activation in the epilogue equals product + silu_mul."""
    x = randn(m, k, dtype=torch.bfloat16, seed=30)
    w = randn(2 * inter, k, dtype=torch.bfloat16, seed=31, scale=0.05)
    b = randn(2 * inter, dtype=torch.bfloat16, seed=32) if bias else None
    got = K().linear_stream(x, w, b, silu_pairs=True)
    assert got.shape == (m, inter) and got.dtype == torch.bfloat16
    products = (x.float() @ w.float().T + (b.float() if bias else 0)).to(torch.bfloat16)
    want = P.silu_mul(products, 8)
    torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=2e-2)
    routed = K().linear_silu_mul(x, w, b, group=8)      # the kernels above for decode-sized batches
    assert torch.equal(got, routed)
    assert K().read_status() == 0


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (8, 6144, 4096), (5, 200, 576), (16, 4096, 1088), (3, 48, 4096)])
@pytest.mark.parametrize("weight_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("gated", [False, True])
def test_residual_stream_kernels(m, n, k, weight_dtype, gated):
    """A sub-layer's exit (product added into the residual, squares left for the norm) and the next
    sub-layer's entry (rows normalised inside the product) equal the separate steps."""
    piece = 64
    x = randn(m, 192, dtype=torch.bfloat16, seed=39)
    w_out = randn(k, 192, dtype=torch.bfloat16, seed=38, scale=0.05)
    b_out = randn(k, dtype=torch.bfloat16, seed=37)
    residual = randn(m, k, dtype=torch.bfloat16, seed=41)
    before = residual.clone()
    pending, sumsq = K().linear_add_residual(x, w_out, b_out, residual)
    assert pending is None and sumsq.shape == (m, -(-k // piece))
    out = (x.float() @ w_out.float().T + b_out.float()).to(torch.bfloat16)
    want_residual = (out.float() + before.float()).to(torch.bfloat16)
    # the product differs from the library's by summation order: allow a bf16 step on the sum
    torch.testing.assert_close(residual.float(), want_residual.float(), rtol=1.6e-2, atol=2e-2)
    torch.testing.assert_close(sumsq.sum(dim=1), residual.float().pow(2).sum(dim=1), rtol=1e-5, atol=1e-5)

    g = (1.0 + 0.2 * randn(k, dtype=torch.float32, seed=42)).to(weight_dtype)
    rows = 2 * n if gated else n
    w = randn(rows, k, dtype=torch.bfloat16, seed=43, scale=0.05)
    b = randn(rows, dtype=torch.bfloat16, seed=44)
    got, same = K().norm_linear(None, residual, g, 1e-5, w, b, silu_group=8 if gated else None, sumsq=sumsq)
    assert same is residual and got.shape == (m, n)
    normed = P.rmsnorm(residual, g, 1e-5)
    products = (normed.float() @ w.float().T + b.float()).to(torch.bfloat16)
    want = P.silu_mul(products, 8) if gated else products
    torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=2e-2)
    again, _ = K().norm_linear(None, residual, g, 1e-5, w, b, silu_group=8 if gated else None, sumsq=sumsq)
    assert torch.equal(got, again)
    # without the squares the same call takes the separate norm kernel: same numbers up to rounding
    plain, _ = K().norm_linear(None, residual, g, 1e-5, w, b, silu_group=8 if gated else None)
    torch.testing.assert_close(got.float(), plain.float(), rtol=1.6e-2, atol=2e-2)
    assert K().read_status() == 0


def test_norm_linear_and_residual_fall_back_for_larger_batches():
    h = randn(200, 128, dtype=torch.bfloat16, seed=40)
    residual = randn(200, 128, dtype=torch.bfloat16, seed=41)
    g = randn(128, dtype=torch.bfloat16, seed=42)
    w = randn(64, 128, dtype=torch.bfloat16, seed=43, scale=0.05)
    want_residual = residual.clone()
    x = P.add_rmsnorm(h, want_residual, g, 1e-6)
    got, new_residual = K().norm_linear(h, residual, g, 1e-6, w)
    assert new_residual is residual and torch.equal(residual, want_residual)   # updated in place
    torch.testing.assert_close(got.float(), x.float() @ w.float().T, rtol=1.6e-2, atol=2e-2)
    pending, sumsq = K().linear_add_residual(h, w, None, randn(200, 64, dtype=torch.bfloat16, seed=45))
    assert sumsq is None and pending.shape == (200, 64)


def test_linear_stream_refuses_what_it_cannot_take():
    x = randn(129, 128, dtype=torch.bfloat16, seed=20)
    w = randn(64, 128, dtype=torch.bfloat16, seed=21)
    with pytest.raises(K().KernelError):
        K().linear_stream(x, w)            # more than 128 rows
    with pytest.raises(K().KernelError):
        K().linear_stream(x[:17], w)   # more than 16 rows
    with pytest.raises(K().KernelError):
        K().linear_stream(x[:4, :72], w[:, :72].contiguous())   # K no multiple of 64
    # the general entry point takes both (library product)
    torch.testing.assert_close(K().linear(x, w).float(), x.float() @ w.float().T, rtol=1.6e-2, atol=2e-2)


def test_linear_stream_takes_row_views():
    """x may be a column slice of a wider buffer (rows 16-byte aligned), as q inside qkv is."""
    full = randn(6, 512 + 256, dtype=torch.bfloat16, seed=23)
    x = full[:, 256:]
    w = randn(300, 512, dtype=torch.bfloat16, seed=24, scale=0.05)
    torch.testing.assert_close(K().linear(x, w).float(), x.float() @ w.float().T, rtol=1.6e-2, atol=2e-2)


def test_kernel_timeline_trace():
    """The trace lists the kernels that ran, with times in order and the blocks' places."""
    x = randn(8, 256, dtype=torch.bfloat16, seed=1)
    w = randn(640, 256, dtype=torch.bfloat16, seed=2, scale=0.05)
    g = randn(256, dtype=torch.bfloat16, seed=3)
    K().linear_stream(x, w)                                   # warm: the library is loaded, buffers exist
    K().trace_start(DEV, capacity=4096, every_block=True)
    K().rmsnorm(x, g, 1e-5)
    K().linear_stream(x, w)
    events = K().trace_stop()
    assert K().trace_stop() == []                             # stopped: nothing more to read
    names = [e["kernel"] for e in events]
    assert "rmsnorm" in names and "gemm_stream" in names
    blocks = [e for e in events if e["kernel"] == "gemm_stream"]
    assert sorted(e["index"] for e in blocks) == list(range(len(blocks)))   # every block once
    assert {e["block"] for e in blocks} >= {"first", "last"}
    for e in events:
        assert e["entry"] <= e["waited"] <= e["exit"] and 0 <= e["sm"] < 1024
    first_norm = min(e["entry"] for e in events if e["kernel"] == "rmsnorm")
    assert all(e["exit"] >= first_norm for e in blocks)       # the product was launched behind the norm
    # with the trace off, kernels record nothing
    K().rmsnorm(x, g, 1e-5)
    assert K().read_status() == 0


def test_a_reported_status_is_raised_without_a_copy():
    """Kernels report into host memory that the device sees: the engine's check after a step costs
    no round trip, and a report becomes an exception."""
    table = randn(10, 32, dtype=torch.float32, seed=1)
    assert K().peek_status() == 0
    K().raise_on_status()                                     # nothing reported: nothing raised
    ids = torch.tensor([3, 12, 5], dtype=torch.int32, device=DEV)   # 12 is outside the table
    K().gather_rows(table, ids)
    torch.cuda.synchronize()
    assert K().peek_status() & 1
    with pytest.raises(K().KernelError, match="token id"):
        K().raise_on_status()
    assert K().peek_status() == 0 and K().read_status() == 0  # the report was cleared
