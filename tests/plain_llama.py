"""Plain, slow implementation of the Llama 3 decoder: whole sequences, no cache, one
function per part, written from the reference's formulas (each function cites file:line
of Baizx98/KVCore).  It shares no code with ``kvcore_b200``: it reads config.json as a
dict and weights as a dict of checkpoint-named tensors, and uses only elementary torch ops.

``tests/golden/`` holds outputs of the reference's own model code on a tiny random model,
against which this file is checked once (tests/test_plain_vs_golden.py); the llama3
frequency scaling, which the reference lacks, rests on its published formula alone.

Precision: everything runs in ``compute`` (float32 or float64).  With ``round_to`` set to
torch.bfloat16 the values are rounded wherever the reference, run in bfloat16, would hold a
bfloat16 tensor, which gives the numbers a faithful bfloat16 run produces.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def _rounder(round_to):
    if round_to is None:
        return lambda x: x
    return lambda x: x.to(round_to).to(x.dtype)


# ---- configuration -------------------------------------------------------------------------
def read_config(folder) -> dict:
    with (Path(folder) / "config.json").open() as handle:
        return json.load(handle)


def head_dim_of(config: dict) -> int:
    # kvcore/model/models/llama3.py:59
    return int(config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"])


def kv_heads_of(config: dict) -> int:
    # kvcore/engine/engine_core.py:164
    return int(config.get("num_key_value_heads") or config["num_attention_heads"])


def rope_theta_of(config: dict) -> float:
    # kvcore/model/layer/rotary_embedding.py:38-49
    params = config.get("rope_parameters")
    if isinstance(params, dict):
        if "rope_theta" in params:
            return float(params["rope_theta"])
        if "theta" in params:
            return float(params["theta"])
    if config.get("rope_theta") is not None:
        return float(config["rope_theta"])
    return 10000.0


def rope_scaling_of(config: dict) -> dict | None:
    scaling = config.get("rope_scaling")
    if not isinstance(scaling, dict):
        scaling = config.get("rope_parameters")
    if not isinstance(scaling, dict):
        return None
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    return None if kind in (None, "default") else dict(scaling, rope_type=kind)


# ---- parts -----------------------------------------------------------------------------------
def rope_inv_freq(config: dict) -> torch.Tensor:
    """[D/2] rotation frequencies in float64.

    Base table: kvcore/model/layer/rotary_embedding.py:62-69 (theta ** (-2j/D)).
    llama3 scaling is absent from the reference; formula of the Llama 3.1 release: with
    wavelength w = 2*pi/f and original context P, keep f if w < P/high, use f/factor if
    w > P/low, else blend ((1-s)*f/factor + s*f) with s = (P/w - low)/(high - low).
    """
    dim = head_dim_of(config)
    theta = rope_theta_of(config)
    freqs = [theta ** (-(2.0 * j) / dim) for j in range(dim // 2)]
    scaling = rope_scaling_of(config)
    if scaling is not None:
        kind = scaling["rope_type"]
        if kind == "linear":
            freqs = [f / float(scaling["factor"]) for f in freqs]
        elif kind == "llama3":
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            original = float(scaling["original_max_position_embeddings"])
            scaled = []
            for f in freqs:
                wavelen = 2.0 * math.pi / f
                if wavelen < original / high:
                    scaled.append(f)
                elif wavelen > original / low:
                    scaled.append(f / factor)
                else:
                    s = (original / wavelen - low) / (high - low)
                    scaled.append((1.0 - s) * f / factor + s * f)
            freqs = scaled
        else:
            raise ValueError(f"plain implementation does not know rope_type {kind!r}")
    return torch.tensor(freqs, dtype=torch.float64)


def embed(token_ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    # kvcore/model/models/llama3.py:178-180
    return table[token_ids.long().to(table.device)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, rnd=lambda t: t) -> torch.Tensor:
    # kvcore/model/layer/rmsnorm.py:22-26 (32-bit inside, cast at the end)
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return rnd(weight * (x * torch.rsqrt(variance + eps)))


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    # kvcore/model/layer/rotary_embedding.py:10-13
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
               rnd=lambda t: t, faithful_tables: bool = False):
    """q [T,H,D], k [T,KVH,D].  kvcore/model/layer/rotary_embedding.py:16-35, 92-98.

    The angle is formed in 32-bit as the reference does (positions.float() * inv_freq.float()).
    ``faithful_tables`` rounds cos/sin themselves as a bfloat16 run of the reference would.
    """
    angles = positions.to(q.device, torch.float32)[:, None] * inv_freq.to(q.device, torch.float32)[None, :]
    emb = torch.cat((angles, angles), dim=-1).to(q.dtype)
    cos, sin = emb.cos()[:, None, :], emb.sin()[:, None, :]
    if faithful_tables:
        cos, sin = rnd(cos), rnd(sin)
    return rnd(q * cos + rotate_half(q) * sin), rnd(k * cos + rotate_half(k) * sin)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int | None = None, rnd=lambda t: t) -> torch.Tensor:
    """q [T,H,D], k,v [T,KVH,D] of ONE sequence -> [T,H,D].

    kvcore/model/attn_backend/torch_paged.py:90-117: query head h reads kv head
    h // (H/KVH); scores over positions <= own, softmax and PV in 32-bit or better.
    ``window``: only the trailing ``window`` positions are visible.
    """
    tokens, heads, _ = q.shape
    group = heads // k.shape[1]
    out = torch.empty_like(q)
    index = torch.arange(tokens, device=q.device)
    visible = index[None, :] <= index[:, None]
    if window is not None:
        visible &= index[None, :] > index[:, None] - window
    for head in range(heads):
        kv_head = head // group
        scores = (q[:, head] @ k[:, kv_head].T) * scale
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, head] = torch.softmax(scores, dim=-1) @ v[:, kv_head]
    return rnd(out)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           rnd=lambda t: t) -> torch.Tensor:
    # kvcore/model/layer/linear.py:6-12 (nn.Linear)
    y = x @ weight.T
    if bias is not None:
        y = y + bias
    return rnd(y)


def swiglu_mlp(x, gate_w, up_w, down_w, gate_b=None, up_b=None, down_b=None, rnd=lambda t: t):
    # kvcore/model/models/llama3.py:42-45; kvcore/model/layer/activation.py:15-17
    gate = linear(x, gate_w, gate_b, rnd)
    up = linear(x, up_w, up_b, rnd)
    hidden = rnd(rnd(torch.nn.functional.silu(gate)) * up)
    return linear(hidden, down_w, down_b, rnd)


# ---- the model -------------------------------------------------------------------------------
def forward_logits(config: dict, weights: dict, token_ids, *, compute=torch.float32,
                   round_to=None, window: int | None = None, rows=None, device=None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence (kvcore/model/models/llama3.py:124-142, 182-200, 245-247).

    ``rows``: only these positions go through the final norm and the head (the result is
    ``[len(rows), V]``); the layers always run the whole sequence.  ``device``: where the same
    elementary operations run (default: where the weights are); a large model is evaluated on the
    GPU in 32- or 64-bit, where torch's matrix products keep full precision (no reduced-precision
    matrix mode is switched on)."""
    rnd = _rounder(round_to)
    if device is not None and torch.device(device).type == "cuda":
        assert not torch.backends.cuda.matmul.allow_tf32, "the plain implementation needs full-precision products"
    w = {name: t.to(device=device, dtype=compute) for name, t in weights.items()}
    if round_to is not None:
        w = {name: rnd(t) for name, t in w.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    tokens = ids.numel()
    heads = int(config["num_attention_heads"])
    kv_heads = kv_heads_of(config)
    dim = head_dim_of(config)
    eps = float(config.get("rms_norm_eps", 1e-6))
    scale = dim ** -0.5  # llama3.py:60
    inv_freq = rope_inv_freq(config)
    positions = torch.arange(tokens)

    def maybe(name):
        return w.get(name)

    h = embed(ids, w["model.embed_tokens.weight"])
    residual = None
    for layer in range(int(config["num_hidden_layers"])):
        p = f"model.layers.{layer}"
        if residual is None:  # llama3.py:130-134
            residual = h
        else:
            residual = rnd(h + residual)
        x = rms_norm(residual, w[f"{p}.input_layernorm.weight"], eps, rnd)
        q = linear(x, w[f"{p}.self_attn.q_proj.weight"], maybe(f"{p}.self_attn.q_proj.bias"), rnd)
        k = linear(x, w[f"{p}.self_attn.k_proj.weight"], maybe(f"{p}.self_attn.k_proj.bias"), rnd)
        v = linear(x, w[f"{p}.self_attn.v_proj.weight"], maybe(f"{p}.self_attn.v_proj.bias"), rnd)
        q = q.view(tokens, heads, dim)
        k = k.view(tokens, kv_heads, dim)
        v = v.view(tokens, kv_heads, dim)
        q, k = apply_rope(q, k, positions, inv_freq, rnd)
        attn = causal_attention(q, k, v, scale, window, rnd).reshape(tokens, heads * dim)
        a = linear(attn, w[f"{p}.self_attn.o_proj.weight"], maybe(f"{p}.self_attn.o_proj.bias"), rnd)
        residual = rnd(a + residual)  # llama3.py:140
        x = rms_norm(residual, w[f"{p}.post_attention_layernorm.weight"], eps, rnd)
        h = swiglu_mlp(
            x,
            w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"], w[f"{p}.mlp.down_proj.weight"],
            maybe(f"{p}.mlp.gate_proj.bias"), maybe(f"{p}.mlp.up_proj.bias"), maybe(f"{p}.mlp.down_proj.bias"),
            rnd,
        )
    last = rnd(h + residual)
    if rows is not None:
        last = last[torch.as_tensor(list(rows), dtype=torch.long, device=last.device)]
    final = rms_norm(last, w["model.norm.weight"], eps, rnd)  # llama3.py:199
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings") else w["lm_head.weight"]
    logits = final @ head.T  # llama3.py:219, 245-247; kept unrounded: the engine emits 32-bit logits
    scale_out = float(config.get("logit_scale", 1.0))
    return logits * scale_out if scale_out != 1.0 else logits


def greedy_generate(config: dict, weights: dict, prompt, steps: int, *, compute=torch.float32):
    """Greedy continuation by re-running the whole sequence each step."""
    tokens = list(prompt)
    out = []
    for _ in range(steps):
        logits = forward_logits(config, weights, tokens, compute=compute)
        token = int(logits[-1].argmax())
        out.append(token)
        tokens.append(token)
    return out


# ---- sampling ----------------------------------------------------------------------------------
def masked_logits(logits: torch.Tensor, temperature: float, top_k: int | None, top_p: float) -> torch.Tensor:
    """Temperature, top-k and top-p as kvcore/sample/sampler.py:122-153; returns logits with
    dropped entries at -inf."""
    x = logits.to(torch.float32) / temperature
    vocab = x.numel()
    order = torch.argsort(x, stable=True)
    sorted_x = x[order]
    if top_k is not None and top_k < vocab:
        threshold = sorted_x[vocab - top_k]
        sorted_x = sorted_x.masked_fill(sorted_x < threshold, float("-inf"))
    if top_p < 1.0:
        probs = torch.softmax(sorted_x, dim=-1)
        cumulative = torch.cumsum(probs, dim=-1)
        drop = cumulative <= 1.0 - top_p
        drop[-1] = False
        sorted_x = sorted_x.masked_fill(drop, float("-inf"))
    out = torch.empty_like(x)
    out[order] = sorted_x
    return out


def load_weights(folder) -> dict:
    """All tensors of a model folder, read with the safetensors package (not the engine's reader)."""
    from safetensors import safe_open

    tensors = {}
    for path in sorted(Path(folder).glob("*.safetensors")):
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            for name in handle.keys():
                tensors[name] = handle.get_tensor(name)
    return tensors
