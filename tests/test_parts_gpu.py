"""Each part of a layer alone against the plain implementation's function of the same role:
norm, rotary encoding, attention mixer (through a cache it fills itself), feed-forward, block,
embedding and head.  Sizes differ from the tiny models'; float32 and bfloat16."""
from __future__ import annotations

import pytest
import torch

import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return dict(rtol=2e-5, atol=2e-5 * scale) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2 * scale)


def fill(part, seed, std=0.05):
    g = torch.Generator().manual_seed(seed)
    for slot in part.weight_slots():
        if slot.init == "ones":
            slot.dest.copy_((1.0 + 0.1 * torch.randn(slot.shape, generator=g)).reshape(slot.dest.shape))
        else:
            slot.dest.copy_((torch.randn(slot.shape, generator=g) * std).reshape(slot.dest.shape))
    part.finalize_weights()
    # in the checkpoint's shape (a slot may scatter its rows inside a packed matrix)
    return {slot.name: slot.dest.detach().float().cpu().reshape(slot.shape) for slot in part.weight_slots()}


def randn(*shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype).to(DEV)


class Ctx:
    """A step context for one or more requests given as (cached length, new tokens)."""

    def __init__(self, lens, table):
        positions, req_index, starts = [], [], [0]
        for r, (c, q) in enumerate(lens):
            positions += list(range(c, c + q))
            req_index += [r] * q
            starts.append(starts[-1] + q)
        self.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
        self.req_index = torch.tensor(req_index, dtype=torch.int32, device=DEV)
        self.query_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        self.context_lens = torch.tensor([c for c, _ in lens], dtype=torch.int32, device=DEV)
        self.num_reqs, self.num_tokens = len(lens), len(positions)
        self.max_query_len = max(q for _, q in lens)
        self.max_seq_len = max(c + q for c, q in lens)
        self.max_seq_len_bound = self.max_seq_len
        self._table = table
        self._shared = {}

    def block_table(self, group):
        return self._table

    def shared(self, key, make):
        if key not in self._shared:
            self._shared[key] = make()
        return self._shared[key]


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from kvcore_b200.parts.norm import RMSNorm

    part = RMSNorm(size=200, eps=3e-6, name="n", dtype=dtype, device=DEV)
    w = fill(part, 1)["n.weight"]
    h, res = randn(9, 200, dtype=dtype, seed=2), randn(9, 200, dtype=dtype, seed=3)
    want_plain = pl.rms_norm(h.float().cpu(), w.to(dtype).float(), 3e-6)
    torch.testing.assert_close(part.forward(h).float().cpu(), want_plain, **tol(dtype, 4))
    total = (h.float() + res.float()).to(dtype).float().cpu()
    y, new_res = part.forward_residual(h, res)
    assert new_res is res and torch.equal(res.float().cpu(), total)
    torch.testing.assert_close(y.float().cpu(), pl.rms_norm(total, w.to(dtype).float(), 3e-6), **tol(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
def test_rotary_part(dtype):
    from kvcore_b200.parts.rope import RotaryEncoding

    config = dict(hidden_size=96 * 3, num_attention_heads=3, head_dim=96, rope_theta=500000.0,
                  rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                    original_max_position_embeddings=64))
    part = RotaryEncoding(head_dim=96, theta=500000.0, rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                          high_freq_factor=4.0, original_max_position_embeddings=64, dtype=dtype, device=DEV)
    ctx = Ctx([(100, 5), (0, 3)], None)
    q, k = randn(8, 3, 96, dtype=dtype, seed=4), randn(8, 1, 96, dtype=dtype, seed=5)
    want_q, want_k = pl.apply_rope(q.float().cpu(), k.float().cpu(), ctx.positions.cpu(), pl.rope_inv_freq(config))
    part.apply(q, k, ctx)
    torch.testing.assert_close(q.float().cpu(), want_q, **tol(dtype, 4))
    torch.testing.assert_close(k.float().cpu(), want_k, **tol(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,window", [(6, 2, 80, None), (4, 4, 128, None), (8, 2, 64, 37)])
def test_attention_mixer_part(dtype, heads, kv_heads, dim, window):
    """The mixer fills its cache in two portions and must equal whole-sequence plain attention."""
    from kvcore_b200.config.model_spec import PartSpec
    from kvcore_b200.engine.step import LayerCache
    from kvcore_b200.parts.attention import PagedAttention

    hidden, tokens, page = 136, 150, 16
    position = PartSpec("rope", dict(head_dim=dim, theta=10000.0))
    part = PagedAttention(hidden_size=hidden, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                          scale=dim ** -0.5, name="a", bias=True, sliding_window=window, position=position,
                          dtype=dtype, device=DEV)
    w = {k: v.to(dtype).float() for k, v in fill(part, 6).items()}
    x = randn(tokens, hidden, dtype=dtype, seed=7)
    pages = -(-tokens // page)
    table = (torch.randperm(pages) + 1).to(torch.int32).view(1, pages).to(DEV)
    k_cache = torch.zeros(pages + 1, kv_heads, page, dim, dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    cache = LayerCache(group=0, planes=(k_cache, v_cache), owner=True, state=None, page_size=page)
    first = 97
    out = torch.cat([part.forward(x[:first].contiguous(), Ctx([(0, first)], table), cache),
                     part.forward(x[first:].contiguous(), Ctx([(first, tokens - first)], table), cache)])
    xf = x.float().cpu()
    q = pl.linear(xf, w["a.q_proj.weight"], w["a.q_proj.bias"]).view(tokens, heads, dim)
    k = pl.linear(xf, w["a.k_proj.weight"], w["a.k_proj.bias"]).view(tokens, kv_heads, dim)
    v = pl.linear(xf, w["a.v_proj.weight"], w["a.v_proj.bias"]).view(tokens, kv_heads, dim)
    config = dict(hidden_size=heads * dim, num_attention_heads=heads, head_dim=dim, rope_theta=10000.0)
    q, k = pl.apply_rope(q, k, torch.arange(tokens), pl.rope_inv_freq(config))
    attn = pl.causal_attention(q, k, v, dim ** -0.5, window).reshape(tokens, heads * dim)
    want = pl.linear(attn, w["a.o_proj.weight"], w["a.o_proj.bias"])
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype, 2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,inter,tokens", [
    (120, 200, 11),    # runs of 8 gate / 8 up rows, the library product (K no multiple of 64)
    (120, 100, 11),    # an intermediate size that is no multiple of 8: gate and up as halves
    (128, 208, 3),     # decode-sized: the streaming kernel with the activation in its epilogue
    (256, 1000, 16),
])
def test_swiglu_part(dtype, hidden, inter, tokens):
    from kvcore_b200.parts.mlp import SwiGLU

    part = SwiGLU(hidden_size=hidden, intermediate_size=inter, name="m", bias=True, dtype=dtype, device=DEV)
    assert part.group == (8 if inter % 8 == 0 else 0)
    w = {k: v.to(dtype).float() for k, v in fill(part, 8).items()}
    x = randn(tokens, hidden, dtype=dtype, seed=9)
    want = pl.swiglu_mlp(x.float().cpu(), w["m.gate_proj.weight"], w["m.up_proj.weight"], w["m.down_proj.weight"],
                         w["m.gate_proj.bias"], w["m.up_proj.bias"], w["m.down_proj.bias"])
    torch.testing.assert_close(part.forward(x, None).float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from kvcore_b200.parts.embedding import LMHead, TokenEmbedding

    emb = TokenEmbedding(vocab_size=301, hidden_size=72, name="e", dtype=dtype, device=DEV)
    w = fill(emb, 10)["e.weight"].to(dtype).float()
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    got = emb.forward(ids)
    assert torch.equal(got.float().cpu(), pl.embed(ids.cpu(), w))
    tied = LMHead(vocab_size=301, hidden_size=72, name="h", tied_to="e", tied_weight=emb.weight, logit_scale=0.25,
                  dtype=dtype, device=DEV)
    assert tied.weight_slots() == [] and tied.ignorable_tensor_names() == ["h.weight"]
    logits = tied.forward(got)
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu(), (got.float().cpu() @ w.T) * 0.25, **tol(dtype))
    free = LMHead(vocab_size=301, hidden_size=72, name="h", dtype=dtype, device=DEV)
    assert [s.name for s in free.weight_slots()] == ["h.weight"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,tokens", [("C", 40), ("D", 40), ("D", 5), ("E", 8)])
def test_block_part(dtype, name, tokens):
    """One pre-norm block with deferred residual: (h, residual) in, (h, residual) out.  Decode-sized
    bf16 batches of widths that are multiples of 64 take the fused path, whose output has already
    joined the residual."""
    from kvcore_b200.config import LlamaConfig
    from kvcore_b200.engine.step import LayerCache
    from kvcore_b200.parts.block import PreNormResidualBlock
    import replay_cases as rc

    from kvcore_b200.parts.base import Summed

    raw = dict(rc.TINY_CONFIGS[name])
    raw.pop("rope_scaling", None)
    layer = LlamaConfig.from_dict(raw).to_model_spec().layers[1]
    part = PreNormResidualBlock(layer=layer, dtype=dtype, device=DEV)
    w = {k: v.to(dtype).float() for k, v in fill(part, 11).items()}
    page = 16
    heads, kvh, dim = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
    table = torch.tensor([[2, 1, 3]], dtype=torch.int32, device=DEV)
    cache = LayerCache(0, (torch.zeros(4, kvh, page, dim, dtype=dtype, device=DEV),
                           torch.zeros(4, kvh, page, dim, dtype=dtype, device=DEV)), True, None, page)
    h, res = randn(tokens, raw["hidden_size"], dtype=dtype, seed=12), randn(tokens, raw["hidden_size"], dtype=dtype, seed=13)
    h0, r0 = h.float().cpu(), res.float().cpu()
    out_h, out_res = part.forward(h, res, Ctx([(0, tokens)], table), cache)
    p = "model.layers.1"
    residual = h0 + r0
    x = pl.rms_norm(residual, w[f"{p}.input_layernorm.weight"], raw["rms_norm_eps"])
    q = pl.linear(x, w[f"{p}.self_attn.q_proj.weight"]).view(tokens, heads, dim)
    k = pl.linear(x, w[f"{p}.self_attn.k_proj.weight"]).view(tokens, kvh, dim)
    v = pl.linear(x, w[f"{p}.self_attn.v_proj.weight"]).view(tokens, kvh, dim)
    q, k = pl.apply_rope(q, k, torch.arange(tokens), pl.rope_inv_freq(raw))
    a = pl.linear(pl.causal_attention(q, k, v, dim ** -0.5).reshape(tokens, heads * dim), w[f"{p}.self_attn.o_proj.weight"])
    residual = a + residual
    x = pl.rms_norm(residual, w[f"{p}.post_attention_layernorm.weight"], raw["rms_norm_eps"])
    want_h = pl.swiglu_mlp(x, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"], w[f"{p}.mlp.down_proj.weight"])
    import kvcore_b200.kernels.api as api
    stream_rows = api.STREAM_AUTO_ROWS
    if isinstance(out_h, Summed):
        assert dtype == torch.bfloat16 and tokens <= stream_rows and out_h.sumsq is not None
        torch.testing.assert_close(out_res.float().cpu(), residual + want_h, **tol(dtype, 4))
        torch.testing.assert_close(out_h.sumsq.sum(dim=1).cpu(), out_res.float().pow(2).sum(dim=1).cpu(),
                                   rtol=1e-4, atol=1e-4)
    else:
        assert not (dtype == torch.bfloat16 and tokens <= stream_rows and raw["hidden_size"] % 64 == 0)
        torch.testing.assert_close(out_res.float().cpu(), residual, **tol(dtype, 4))
        torch.testing.assert_close(out_h.float().cpu(), want_h, **tol(dtype, 2))
