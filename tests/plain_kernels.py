"""Plain PyTorch statement of every kernel op, with the signatures of ``kvcore_b200.kernels``.

Two uses, both in tests only: (1) each CUDA kernel is compared alone against the function
of the same name here; (2) ``install(monkeypatch)`` swaps these in for the CUDA wrappers so
that the host side (step function, cache manager, scheduler, entry point) can be exercised
on a machine without a GPU.  The product never imports this file.
"""
from __future__ import annotations


import numpy as np
import torch


def require_device(device) -> None:
    return None


def ensure_built(verbose: bool = False) -> str:
    return "plain"


def read_status(reset: bool = True) -> int:
    return 0


def peek_status() -> int:
    return 0


def raise_on_status() -> None:
    return None


def check_attention_shape(num_heads, num_kv_heads, head_dim, dtype) -> None:
    from kvcore_b200.kernels.api import check_attention_shape as real

    real(num_heads, num_kv_heads, head_dim, dtype)


def gather_rows(table, ids, out=None):
    return table[ids.long()]


def feed_tokens(token_ids, source, sampled):
    take = source >= 0
    token_ids[take] = sampled[source[take].long()]


def rmsnorm(x, weight, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (weight.float() * y).to(x.dtype)


def add_rmsnorm(h, residual, weight, eps):
    residual.copy_((h.float() + residual.float()).to(h.dtype))
    return rmsnorm(residual, weight, eps)


def silu_mul(gate_up, group=0):
    inter = gate_up.shape[1] // 2
    if group:
        runs = gate_up.reshape(gate_up.shape[0], inter // group, 2, group)
        gate, up = runs[:, :, 0].reshape(-1, inter).float(), runs[:, :, 1].reshape(-1, inter).float()
    else:
        gate, up = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    act = torch.nn.functional.silu(gate).to(gate_up.dtype).float()
    return (act * up).to(gate_up.dtype)


def _rotate(x, positions, inv_freq):
    half = x.shape[-1] // 2
    angles = positions.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)
    cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1).to(x.dtype)


def rope_inplace(q, k, positions, inv_freq):
    q.copy_(_rotate(q, positions, inv_freq))
    if k is not None:
        k.copy_(_rotate(k, positions, inv_freq))


def rope_table(positions, inv_freq):
    angles = positions.to(torch.float32)[:, None] * inv_freq[None, :].to(torch.float32)
    return torch.stack((angles.cos(), angles.sin()), dim=-1)


def _rotate_with(x, cos_sin):
    half = x.shape[-1] // 2
    cos, sin = cos_sin[:, None, :, 0], cos_sin[:, None, :, 1]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1).to(x.dtype)


def rope_kv_write(qkv, positions, req_index, cos_sin, table, k_cache, v_cache,
                  num_heads, num_kv_heads, head_dim, *, write_kv=True):
    tokens = qkv.shape[0]
    q_size, kv_size = num_heads * head_dim, num_kv_heads * head_dim
    q = qkv[:, :q_size].view(tokens, num_heads, head_dim)
    k = qkv[:, q_size:q_size + kv_size].view(tokens, num_kv_heads, head_dim)
    v = qkv[:, q_size + kv_size:].view(tokens, num_kv_heads, head_dim)
    if cos_sin is not None:
        q.copy_(_rotate_with(q, cos_sin))
        k.copy_(_rotate_with(k, cos_sin))
    if write_kv:
        page_size = k_cache.shape[2]
        for t in range(tokens):
            pos = int(positions[t])
            page = int(table[int(req_index[t]), pos // page_size])
            assert page > 0, "write through the null page"
            k_cache[page, :, pos % page_size, :] = k[t]
            v_cache[page, :, pos % page_size, :] = v[t]


def paged_attention(qkv, k_cache, v_cache, table, ctx, num_heads, num_kv_heads, head_dim, scale, window,
                    *, force_general=False, num_splits=None, use_tma=True, use_tc5=True, cos_sin=None,
                    write_kv=None):
    if write_kv is not None:   # the call also rotates q, k and writes this step's k, v
        rope_kv_write(qkv, ctx.positions, ctx.req_index, cos_sin, table, k_cache, v_cache,
                      num_heads, num_kv_heads, head_dim, write_kv=write_kv)
    return paged_attention_plain(qkv, k_cache, v_cache, table, ctx.positions, ctx.req_index,
                                 num_heads, num_kv_heads, head_dim, scale, window)


def paged_attention_plain(qkv, k_cache, v_cache, table, positions, req_index,
                          num_heads, num_kv_heads, head_dim, scale, window):
    tokens = qkv.shape[0]
    page_size = k_cache.shape[2]
    group = num_heads // num_kv_heads
    out = torch.empty((tokens, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    q = qkv[:, : num_heads * head_dim].view(tokens, num_heads, head_dim).float()
    for t in range(tokens):
        pos = int(positions[t])
        first = 0 if not window else max(0, pos - window + 1)
        keys = torch.arange(first, pos + 1, device=qkv.device)
        pages = table[int(req_index[t])].long()[keys // page_size]
        assert bool((pages > 0).all()), "read through the null page"
        offsets = keys % page_size
        k = k_cache[pages, :, offsets, :].float()  # [n, KVH, D]
        v = v_cache[pages, :, offsets, :].float()
        for h in range(num_heads):
            g = h // group
            scores = (k[:, g, :] @ q[t, h]) * scale
            probs = torch.softmax(scores, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = (probs @ v[:, g, :]).to(qkv.dtype)
    return out


def linear(x, weight, bias=None, *, out_dtype=None):
    y = x.float() @ weight.float().T
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype or x.dtype)


def linear_silu_mul(x, weight, bias=None, *, group=0):
    return silu_mul(linear(x, weight, bias), group)


def norm_linear(h, residual, norm_weight, eps, weight, bias=None, *, silu_group=None, sumsq=None):
    if h is None:
        x = rmsnorm(residual, norm_weight, eps)
    elif residual is None:
        x, residual = rmsnorm(h, norm_weight, eps), h
    else:
        x = add_rmsnorm(h, residual, norm_weight, eps)
    out = linear(x, weight, bias) if silu_group is None else linear_silu_mul(x, weight, bias, group=silu_group)
    return out, residual


def linear_add_residual(x, weight, bias, residual):
    return linear(x, weight, bias), None


# ---- sampling: the same counter-based noise as the CUDA kernel --------------------------------
def philox4x32_10(counter, key):
    c = [np.uint64(x) for x in counter]
    k = [np.uint64(x) for x in key]
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c[0]
        p1 = np.uint64(0xCD9E8D57) * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [(hi1 ^ c[1] ^ k[0]) & mask, lo1, (hi0 ^ c[3] ^ k[1]) & mask, lo0]
        k = [(k[0] + np.uint64(0x9E3779B9)) & mask, (k[1] + np.uint64(0xBB67AE85)) & mask]
    return [int(x) for x in c]


def exponential_noise(vocab: int, seed: int, token_index: int) -> np.ndarray:
    """q[i] ~ Exp(1) exactly as the kernel draws it (float32 arithmetic)."""
    q = np.empty(vocab, dtype=np.float32)
    lo, hi = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for group in range((vocab + 3) // 4):
        r = philox4x32_10((group, token_index, 0, 0), (lo, hi))
        for j in range(4):
            i = group * 4 + j
            if i < vocab:
                u = (np.float32(r[j]) + np.float32(0.5)) * np.float32(2.3283064365386963e-10)
                u = min(u, np.float32(0.99999994))
                q[i] = -np.log(u, dtype=np.float32)
    return q


def sample_row(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, seed: int,
               token_index: int, eps: float = 1e-5):
    """Returns (token, scores) where scores[i] = (x_i - max) - log(q_i) over kept entries."""
    from plain_llama import masked_logits

    if temperature < eps:
        return int(torch.argmax(logits)), None
    vocab = logits.numel()
    x = masked_logits(logits, temperature, top_k if top_k < vocab else None, top_p)
    q = torch.from_numpy(exponential_noise(vocab, seed, token_index))
    scores = (x - x.max()) - torch.log(q)
    return int(torch.argmax(scores)), scores


def sample(logits, packed_params, eps):
    out = torch.empty(logits.shape[0], dtype=torch.int32)
    for row in range(logits.shape[0]):
        temperature, top_k, top_p, lo, hi, index = packed_params[row].tolist()
        seed = int(lo) | (int(hi) << 32)
        out[row], _ = sample_row(logits[row].float().cpu(), temperature, int(top_k), top_p, seed, int(index), eps)
    return out.to(logits.device)


_NAMES = [
    "require_device", "ensure_built", "read_status", "peek_status", "raise_on_status", "check_attention_shape", "gather_rows", "feed_tokens", "rmsnorm",
    "add_rmsnorm", "silu_mul", "rope_inplace", "rope_table", "rope_kv_write", "paged_attention", "linear", "linear_silu_mul", "norm_linear", "linear_add_residual", "sample",
]


def install(monkeypatch) -> None:
    """Replace the CUDA wrappers of ``kvcore_b200.kernels`` by the functions of this file."""
    import kvcore_b200.kernels as K

    module = globals()
    for name in _NAMES:
        monkeypatch.setattr(K, name, module[name])
