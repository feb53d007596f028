"""Python face of the CUDA library: one function per kernel, taking torch tensors.

Each wrapper checks device, dtype, contiguity and sizes, then calls the exported C entry
point with raw device pointers on torch's current stream.  There is no CPU path and no
fallback: a tensor that is not on a CUDA device, or a library that cannot be built or
loaded, raises.  Library matrix products (cuBLAS through torch) stand in for the bf16
linear layers, as the reference uses a library for them (kvcore/model/layer/linear.py:6-12).
"""
from __future__ import annotations

import ctypes
import os
from typing import Any

import torch

from . import build as _build

_F32, _BF16 = 0, 1
_lib: ctypes.CDLL | None = None
_vp = ctypes.c_void_p
_int = ctypes.c_int
_ll = ctypes.c_longlong
_float = ctypes.c_float


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or its launch failed."""


def ensure_built(verbose: bool = False) -> str:
    """Build (if needed) and load the CUDA library; returns its path."""
    global _lib
    if _lib is not None:
        return _lib._name
    path = _build.build(verbose=verbose)
    lib = ctypes.CDLL(str(path))
    lib.kvb_last_error.restype = ctypes.c_char_p
    lib.kvb_status_word.restype = _vp
    signatures: dict[str, list[Any]] = {
        "kvb_gather_rows": [_vp, _vp, _vp, _int, _int, _int, _int, _vp],
        "kvb_rmsnorm": [_vp, _vp, _vp, _vp, _int, _int, _float, _int, _int, _vp],
        "kvb_silu_mul": [_vp, _vp, _int, _int, _int, _int, _vp],
        "kvb_rope_table": [_vp, _vp, _vp, _int, _int, _vp],
        "kvb_rope_kv_write": [_vp, _ll, _vp, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int, _int,
                              _int, _int, _int, _vp],
        "kvb_paged_attention_rows": [_vp, _int, _vp, _int, _vp, _vp, _vp, _int, _vp, _vp, _int, _int,
                                     _int, _int, _int, _int, _float, _int, _int, _vp],
        "kvb_flash_paged_attention": [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int,
                                      _int, _int, _int, _int, _float, _int, _int, _vp, _vp],
        "kvb_make_kv_tensor_map": [_vp, _vp, _ll, _int, _int, _int],
        "kvb_flash_decode_tma": [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int, _int,
                                 _int, _int, _int, _float, _int, _int, _vp, _vp, _vp, _vp, _vp, _int, _vp],
        "kvb_make_kv_half_tensor_map": [_vp, _vp, _ll, _int, _int, _int],
        "kvb_flash_prefill_tc5": [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int, _int, _int,
                                  _int, _int, _int, _float, _int, _vp],
        "kvb_gemm_f32": [_vp, _vp, _vp, _vp, _int, _int, _int, _ll, _ll, _vp],
        "kvb_gemm_stream_bf16": [_vp, _int, _ll, _vp, _ll, _vp, _vp, _int, _int, _int, _int, _vp, _int, _float, _vp,
                                 _int, _vp, _vp, _vp, _int, _vp],
        "kvb_sample": [_vp, _vp, _vp, _int, _int, _float, _vp],
        "kvb_feed_tokens": [_vp, _vp, _vp, _int, _int, _vp],
        "kvb_read_status": [_int, ctypes.POINTER(ctypes.c_int)],
    }
    for name, argtypes in signatures.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _int
    lib.kvb_set_pdl.argtypes = [_int]
    lib.kvb_set_pdl.restype = None
    lib.kvb_peek_status.argtypes = []
    lib.kvb_peek_status.restype = _int
    # Kernels of this library overlap their start with the end of the kernel in front of them
    # (programmatic dependent launch); KVCORE_B200_SERIAL_LAUNCH=1 switches that off.
    lib.kvb_set_pdl(0 if os.environ.get("KVCORE_B200_SERIAL_LAUNCH") == "1" else 1)
    lib.kvb_gemm_stream_scratch_floats.argtypes = [_int]
    lib.kvb_gemm_stream_scratch_floats.restype = _ll
    lib.kvb_gemm_stream_norm_max_k.argtypes = []
    lib.kvb_gemm_stream_norm_max_k.restype = _int
    lib.kvb_gemm_stream_scratch_marker.argtypes = []
    lib.kvb_gemm_stream_scratch_marker.restype = ctypes.c_uint
    _lib = lib
    return str(path)


def library_is_loaded() -> bool:
    return _lib is not None


def require_device(device: torch.device | str) -> None:
    """Fail loudly unless ``device`` is a usable CUDA device and the library loads."""
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelError(f"kvcore_b200 runs on CUDA devices only, got device {device}")
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available; kvcore_b200 has no CPU path")
    ensure_built()
    with torch.cuda.device(device):
        if not _lib.kvb_status_word():
            raise KernelError("cannot allocate the device status word")


launch_count = 0  # kernels of this library launched so far (read by the benchmark)


def _call(name: str, *args: Any, kernels: int = 1) -> None:
    """Run entry point ``name``, which launches ``kernels`` kernels."""
    global launch_count
    if _lib is None:
        ensure_built()
    launch_count += kernels
    code = getattr(_lib, name)(*args)
    if code != 0:
        raise KernelError(f"{name}: {_lib.kvb_last_error().decode()}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"unsupported tensor dtype {t.dtype}: kernels take float32 or bfloat16")


def _check(t: torch.Tensor, name: str, *, dtype: torch.dtype | None = None, contiguous: bool = True) -> None:
    if t.device.type != "cuda":
        raise KernelError(f"{name} must be on a CUDA device, got {t.device}: there is no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def read_status(reset: bool = True) -> int:
    """Status bits set by kernels (1 bad token id, 2 bad page id, 4 bounded wait ran out)."""
    out = ctypes.c_int(0)
    _call("kvb_read_status", int(reset), ctypes.byref(out))
    if out.value & 4:
        # a kernel gave up a wait: the hand-over areas of the streaming kernels may hold parts that
        # nobody took; put them back into their state between launches
        for scratch in _stream_scratch.values():
            scratch.view(torch.int32).fill_(int(_lib.kvb_gemm_stream_scratch_marker()))
        for counters in _decode_work_counters.values():
            counters.zero_()
    return out.value


STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a page id outside the cache",
               4: "a bounded wait inside a kernel ran out"}


def peek_status() -> int:
    """The status bits reported by the kernels that have finished, without waiting for any: free to
    call after the caller has synchronised on its own (0 when the library is not loaded)."""
    if _lib is None:
        return 0
    return int(_lib.kvb_peek_status())


def raise_on_status() -> None:
    """Raise ``KernelError`` if a finished kernel reported a problem (and clear the report)."""
    if peek_status():
        bits = read_status(reset=True)
        what = "; ".join(text for bit, text in STATUS_BITS.items() if bits & bit) or f"status {bits}"
        raise KernelError(f"a kernel reported: {what}")


# ---- shape policy -------------------------------------------------------------------------------
def check_attention_shape(num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> None:
    """Refuse, with a clear error, head shapes the attention kernels do not take."""
    if head_dim <= 0 or head_dim % 2 or head_dim > 256:
        raise ValueError(f"head_dim must be even and at most 256, got {head_dim}")
    if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
        raise ValueError(
            f"num_heads {num_heads} must be a positive multiple of num_kv_heads {num_kv_heads}"
        )
    if dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"attention runs in float32 or bfloat16, got {dtype}")


# ---- kernels --------------------------------------------------------------------------------------
def gather_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[i] = table[ids[i]]`` for int32 ``ids``; used for the embedding and for logits rows."""
    _check(table, "table")
    _check(ids, "ids", dtype=torch.int32)
    if table.dim() != 2:
        raise KernelError(f"table must be [rows, width], got {tuple(table.shape)}")
    count, (rows, width) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((count, width), dtype=table.dtype, device=table.device)
    _call("kvb_gather_rows", out.data_ptr(), table.data_ptr(), ids.data_ptr(), count, width, rows,
          _dtype_code(table), _stream())
    return out


def feed_tokens(token_ids: torch.Tensor, source: torch.Tensor, sampled: torch.Tensor) -> None:
    """``token_ids[t] = sampled[source[t]]`` wherever ``source[t] >= 0`` (all int32, in place): the
    ids of a step that was packed before the step in front had been read back."""
    _check(token_ids, "token_ids", dtype=torch.int32)
    _check(source, "source", dtype=torch.int32)
    _check(sampled, "sampled", dtype=torch.int32)
    if source.numel() != token_ids.numel():
        raise KernelError(f"one source per token id is needed, got {source.numel()} for {token_ids.numel()}")
    _call("kvb_feed_tokens", token_ids.data_ptr(), source.data_ptr(), sampled.data_ptr(), token_ids.numel(),
          sampled.numel(), _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _check(x, "x")
    _check(weight, "weight")
    rows, width = x.shape
    if weight.numel() != width:
        raise KernelError(f"norm weight has {weight.numel()} entries for rows of width {width}")
    out = torch.empty_like(x)
    _call("kvb_rmsnorm", out.data_ptr(), None, x.data_ptr(), weight.data_ptr(), rows, width,
          float(eps), _dtype_code(x), _dtype_code(weight), _stream())
    return out


def add_rmsnorm(h: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``residual += h`` in place, returns ``norm(residual) * weight``."""
    _check(h, "h")
    _check(residual, "residual", dtype=h.dtype)
    _check(weight, "weight")
    if h.shape != residual.shape:
        raise KernelError(f"h {tuple(h.shape)} and residual {tuple(residual.shape)} differ in shape")
    rows, width = h.shape
    if weight.numel() != width:
        raise KernelError(f"norm weight has {weight.numel()} entries for rows of width {width}")
    out = torch.empty_like(h)
    _call("kvb_rmsnorm", out.data_ptr(), residual.data_ptr(), h.data_ptr(), weight.data_ptr(), rows,
          width, float(eps), _dtype_code(h), _dtype_code(weight), _stream())
    return out


def silu_mul(gate_up: torch.Tensor, group: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` of a packed ``[T, 2I]`` tensor.

    ``group == 0``: gate is ``gate_up[:, :I]``, up is ``gate_up[:, I:]``.  ``group > 0``: gate and
    up columns alternate in runs of ``group`` (gate 0..g-1, up 0..g-1, gate g..2g-1, ...)."""
    _check(gate_up, "gate_up")
    rows, two_inter = gate_up.shape
    if two_inter % 2:
        raise KernelError(f"gate_up must have an even width, got {two_inter}")
    inter = two_inter // 2
    if group < 0 or (group and inter % group):
        raise KernelError(f"silu_mul: group {group} does not divide the width {inter}")
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _call("kvb_silu_mul", out.data_ptr(), gate_up.data_ptr(), rows, inter, group, _dtype_code(gate_up), _stream())
    return out


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """``[T, D/2, 2]`` float32 (cos, sin) of ``float(position) * inv_freq``: made once per step."""
    _check(positions, "positions", dtype=torch.int32)
    _check(inv_freq, "inv_freq", dtype=torch.float32)
    tokens, half = positions.numel(), inv_freq.numel()
    table = torch.empty((tokens, half, 2), dtype=torch.float32, device=positions.device)
    _call("kvb_rope_table", table.data_ptr(), positions.data_ptr(), inv_freq.data_ptr(), tokens, half, _stream())
    return table


def rope_kv_write(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    req_index: torch.Tensor,
    cos_sin: torch.Tensor | None,
    table: torch.Tensor | None,
    k_cache: torch.Tensor | None,
    v_cache: torch.Tensor | None,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    *,
    write_kv: bool = True,
) -> None:
    """Rotate q and k of ``qkv [T, (H+2KVH)*D]`` in place with the ``rope_table`` values
    ``cos_sin`` (``None``: no rotation) and write k, v into their pages."""
    _check(qkv, "qkv", contiguous=False)
    _check(positions, "positions", dtype=torch.int32)
    _check(req_index, "req_index", dtype=torch.int32)
    tokens = qkv.shape[0]
    if qkv.stride(1) != 1:
        raise KernelError("qkv rows must be contiguous")
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv width {qkv.shape[1]} does not match the head layout")
    if cos_sin is not None:
        _check(cos_sin, "cos_sin", dtype=torch.float32)
        if tuple(cos_sin.shape) != (tokens, head_dim // 2, 2):
            raise KernelError(f"cos_sin has shape {tuple(cos_sin.shape)} for {tokens} tokens of head_dim {head_dim}")
    k_ptr = v_ptr = table_ptr = None
    table_stride = page_size = num_pages = 0
    if write_kv:
        if k_cache is None or v_cache is None or table is None:
            raise KernelError("a cache write needs k_cache, v_cache and a block table")
        _check(k_cache, "k_cache", dtype=qkv.dtype)
        _check(v_cache, "v_cache", dtype=qkv.dtype)
        _check(table, "block table", dtype=torch.int32, contiguous=False)
        num_pages, kvh, page_size, d = k_cache.shape
        if (kvh, d) != (num_kv_heads, head_dim) or v_cache.shape != k_cache.shape:
            raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match the head layout")
        if table.stride(1) != 1:
            raise KernelError("block table rows must be contiguous")
        k_ptr, v_ptr, table_ptr = k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr()
        table_stride = table.stride(0)
    if cos_sin is None and not write_kv:
        return
    _call("kvb_rope_kv_write", qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), req_index.data_ptr(),
          None if cos_sin is None else cos_sin.data_ptr(), table_ptr, table_stride, k_ptr, v_ptr,
          tokens, num_heads, num_kv_heads, head_dim, page_size, num_pages, _dtype_code(qkv), _stream())


def rope_inplace(q: torch.Tensor, k: torch.Tensor | None, positions: torch.Tensor, inv_freq: torch.Tensor) -> None:
    """Rotate ``q [T, H, D]`` (and ``k [T, KVH, D]``) in place without touching a cache; rows may
    be views into a wider buffer as long as heads are contiguous."""
    cos_sin = rope_table(positions, inv_freq)
    for x in (q, k):
        if x is None:
            continue
        _check(x, "q/k", contiguous=False)
        tokens, heads, head_dim = x.shape
        if x.stride(2) != 1 or x.stride(1) != head_dim:
            raise KernelError("rope_inplace: heads must be contiguous within a row")
        if inv_freq.numel() != head_dim // 2:
            raise KernelError(f"inv_freq has {inv_freq.numel()} entries for head_dim {head_dim}")
        _call("kvb_rope_kv_write", x.data_ptr(), x.stride(0), positions.data_ptr(), positions.data_ptr(),
              cos_sin.data_ptr(), None, 0, None, None, tokens, heads, 0, head_dim, 0, 0,
              _dtype_code(x), _stream())


_sm_counts: dict[int, int] = {}
_FLASH_CTAS_PER_SM = 3


def sm_count(device: torch.device | str | int | None = None) -> int:
    """Multiprocessors of ``device`` (default: the current CUDA device), asked from the driver once
    per device.  Grids, split counts and the scratch of the streaming kernels are sized from it."""
    if device is None:
        index = torch.cuda.current_device()
    elif isinstance(device, int):
        index = device
    else:
        device = torch.device(device)
        if device.type != "cuda":
            raise KernelError(f"kvcore_b200 runs on CUDA devices only, got device {device}")
        index = torch.cuda.current_device() if device.index is None else device.index
    count = _sm_counts.get(index)
    if count is None:
        count = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return count


def flash_attention_supported(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether the tensor-core kernel takes this shape (else the general kernel runs)."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128


def decode_splits(num_reqs: int, num_kv_heads: int, max_seq_len: int, sms: int | None = None) -> int:
    """How many chunks each request's keys are cut into so that the GPU (``sms`` multiprocessors,
    default: the current device's) is filled."""
    blocks = max(1, num_reqs * num_kv_heads)
    wanted = -(-(sms or sm_count()) * _FLASH_CTAS_PER_SM // blocks)
    longest = max(1, -(-max_seq_len // 256))  # a split of fewer than 256 keys is not worth a block
    return max(1, min(wanted, longest, 64))


def tma_decode_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the TMA-fed decode kernel takes this cache shape."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size in (8, 16, 32, 64)


def decode_splits_tma(num_reqs: int, num_kv_heads: int, max_seq_len: int, sms: int | None = None) -> int:
    """Splits for the TMA decode kernel, which keeps two blocks per SM (measured inside whole steps
    on B200; ``sms``: multiprocessors, default the current device's).

    Up to half a wave of (request, kv head) pairs: as many splits as still fit one wave of blocks,
    at most 16 (the merge grows with them) and at least two 64-key tiles a split (batch 1 at 1,024
    tokens gains 3.6 % with 8 splits over 2, loses with 16; at 8,192 tokens 16 beat 24, 32 and 37).

    More pairs than that: the kernel is bound by memory as long as the last wave is not sparse
    (64 requests x 8 heads = 1.73 waves run at 0.97 of the copy bandwidth unsplit, and 4 splits
    are 1.3 % slower), but a last wave of a few blocks runs no faster than ~0.45 of a full one
    (48 requests at 8,192 tokens: 3 splits -11 % a step; 40 at 4,096: 4 splits -9 %).  So the
    cost of 1 to 4 splits is estimated as full waves + max(rest, 0.45), half a percent a split for
    the merge, and the cheapest is taken."""
    base = max(1, num_reqs * num_kv_heads)
    tiles = max(1, -(-max_seq_len // 64))
    wave = (sms or sm_count()) * TMA_DECODE_BLOCKS_PER_SM
    if base * 2 <= wave:
        return max(1, min(wave // base, tiles // 2, 16))
    best, best_cost = 1, float("inf")
    for splits in (1, 2, 3, 4):
        if splits > 1 and tiles // splits < 4:
            break
        full, rest = divmod(base * splits, wave)
        cost = (full + (max(rest / wave, 0.45) if rest else 0.0)) / splits * (1.0 + 0.005 * (splits - 1))
        if cost < best_cost - 1e-9:
            best, best_cost = splits, cost
    return best


TMA_DECODE_BLOCKS_PER_SM = 2
# more (request, kv head, split) items than blocks fit the GPU at once: blocks stay and share the items
# (KVCORE_B200_DECODE_SHARED_WORK=0: one block an item, whatever their number)
TMA_DECODE_SHARED_WORK = os.environ.get("KVCORE_B200_DECODE_SHARED_WORK", "1") != "0"
_decode_work_counters: dict[torch.device, torch.Tensor] = {}


def _decode_work(device: torch.device) -> torch.Tensor:
    """Two counters through which the blocks of the TMA decode kernel share out their work when there
    is more of it than blocks that fit the GPU at once (zero between launches: the kernel's last
    block puts them back)."""
    counters = _decode_work_counters.get(device)
    if counters is None:
        counters = _decode_work_counters[device] = torch.zeros(2, dtype=torch.int32, device=device)
    return counters

_kv_tensor_maps: dict[tuple, tuple] = {}


def _kv_tensor_map_pair(k_cache: torch.Tensor, v_cache: torch.Tensor, kind: str = "page") -> tuple:
    """Host-side TMA descriptors of one layer's K and V cache, made once per tensor.  ``kind``:
    "page" = one contiguous box per page and head (decode), "half" = boxes of one 64-column half
    of a page (operand tiles of the tcgen05 prefill kernel)."""
    key = (kind, k_cache.data_ptr(), v_cache.data_ptr(), tuple(k_cache.shape))
    maps = _kv_tensor_maps.get(key)
    if maps is None:
        num_pages, kvh, page_size, d = k_cache.shape
        maps = (ctypes.create_string_buffer(128), ctypes.create_string_buffer(128))
        maker = "kvb_make_kv_tensor_map" if kind == "page" else "kvb_make_kv_half_tensor_map"
        for buffer, cache in zip(maps, (k_cache, v_cache)):
            _call(maker, ctypes.addressof(buffer), cache.data_ptr(), num_pages, kvh, page_size, d)
        _kv_tensor_maps[key] = maps
    return maps


def tc5_prefill_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill kernel takes this cache shape."""
    return dtype == torch.bfloat16 and head_dim == 128 and page_size in (8, 16, 32, 64)


def paged_attention(
    qkv: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    table: torch.Tensor,
    ctx,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int | None,
    *,
    force_general: bool = False,
    num_splits: int | None = None,
    use_tma: bool = True,
    use_tc5: bool = True,
    cos_sin: torch.Tensor | None = None,
    write_kv: bool | None = None,
) -> torch.Tensor:
    """Attention of the step's queries (the first ``H*D`` columns of ``qkv``) over the cache.

    Returns ``[T, H*D]``.  ``ctx`` describes the batch: positions and request rows of the
    tokens, and per request its query start and cached length.  bfloat16 with a head size in
    steps of 16 up to 128 runs on the tensor-core kernel (split over the keys for decode
    batches); everything else, and all of float32, runs on the general kernel.

    ``write_kv=None``: q and k in ``qkv`` are rotated already and the cache holds this step's
    keys and values.  Otherwise this call also rotates q and k with the ``rope_table`` values
    ``cos_sin`` (``None``: no rotation) and, if ``write_kv``, writes this step's k and v into
    their pages: inside the decode kernel where that one runs (``qkv`` is then left as it
    was), through ``rope_kv_write`` in front of the other kernels.
    """
    if write_kv is not None:
        group = num_heads // num_kv_heads
        fused = (not force_general and use_tma and flash_attention_supported(qkv.dtype, head_dim)
                 and qkv.stride(0) % 8 == 0 and ctx.max_query_len * group <= 16
                 and tma_decode_supported(qkv.dtype, head_dim, k_cache.shape[2]))
        if not fused:
            rope_kv_write(qkv, ctx.positions, ctx.req_index, cos_sin, table, k_cache, v_cache,
                          num_heads, num_kv_heads, head_dim, write_kv=write_kv)
            cos_sin, write_kv = None, None
        elif cos_sin is not None:
            _check(cos_sin, "cos_sin", dtype=torch.float32)
            if tuple(cos_sin.shape) != (qkv.shape[0], head_dim // 2, 2):
                raise KernelError(f"cos_sin has shape {tuple(cos_sin.shape)} for {qkv.shape[0]} tokens "
                                  f"of head_dim {head_dim}")
    _check(qkv, "qkv", contiguous=False)
    _check(k_cache, "k_cache", dtype=qkv.dtype)
    _check(v_cache, "v_cache", dtype=qkv.dtype)
    _check(table, "block table", dtype=torch.int32, contiguous=False)
    tokens = qkv.shape[0]
    num_pages, kvh, page_size, d = k_cache.shape
    if (kvh, d) != (num_kv_heads, head_dim):
        raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match the head layout")
    out = torch.empty((tokens, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if not force_general and flash_attention_supported(qkv.dtype, head_dim) and qkv.stride(0) % 8 == 0:
        group = num_heads // num_kv_heads
        geometry = (num_heads, num_kv_heads, head_dim, float(scale), int(window or 0))
        # A mixed step (portions of prompts beside single decoded tokens) is two kinds of work: the
        # portions fill query tiles of 128 rows, a decoded token has at most 16 rows a kv head and would
        # leave such a tile almost empty while walking all its keys.  When the batch says how long each
        # request's portion is and stands longest first (the step function packs it so), the two runs of
        # requests go to the kernel made for each.
        lens = getattr(ctx, "host_query_lens", None)
        contexts = getattr(ctx, "host_context_lens", None)
        if (write_kv is None and num_splits is None and lens and contexts and len(lens) == ctx.num_reqs
                and ctx.max_query_len * group > 16):
            long_count = sum(1 for n in lens if n * group > 16)
            if 0 < long_count < ctx.num_reqs and all(n * group > 16 for n in lens[:long_count]):
                for begin, end in ((0, long_count), (long_count, ctx.num_reqs)):
                    part = _RequestRun(ctx, begin, end)
                    _flash_attention_into(out, qkv, k_cache, v_cache, table[begin:end], part, geometry,
                                          None, use_tma, use_tc5, None, None)
                return out
        _flash_attention_into(out, qkv, k_cache, v_cache, table, ctx, geometry, num_splits, use_tma, use_tc5,
                              cos_sin, write_kv)
        return out
    _call("kvb_paged_attention_rows", out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0),
          k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr(), table.stride(0),
          ctx.positions.data_ptr(), ctx.req_index.data_ptr(), tokens, num_heads, num_kv_heads,
          head_dim, page_size, num_pages, float(scale), int(window or 0), _dtype_code(qkv), _stream())
    return out


class _RequestRun:
    """Requests ``[begin, end)`` of a step's batch, as the attention kernels need a batch described:
    views of the per-request arrays (query starts are token offsets into the whole step, so outputs
    land in the rows of the whole step's tensors) and the lengths that size the launch."""

    def __init__(self, ctx, begin: int, end: int) -> None:
        lens, contexts = ctx.host_query_lens[begin:end], ctx.host_context_lens[begin:end]
        self.num_reqs = end - begin
        self.max_query_len = max(lens)
        self.max_seq_len = max(c + n for c, n in zip(contexts, lens))
        self.max_seq_len_bound = 0
        self.query_start = ctx.query_start[begin : end + 1]
        self.context_lens = ctx.context_lens[begin:end]


def _flash_attention_into(out, qkv, k_cache, v_cache, table, ctx, geometry, num_splits, use_tma, use_tc5,
                          cos_sin, write_kv) -> None:
    """The tensor-core attention kernels on one batch (or one run of requests of a batch): the TMA
    decode kernel for at most 16 rows a kv head, the tcgen05 kernel for portions of prompts, the
    ``mma.sync`` kernel for the shapes those two do not take."""
    num_heads, num_kv_heads, head_dim, scale, window = geometry
    num_pages, _, page_size, _ = k_cache.shape
    group = num_heads // num_kv_heads
    split_mode = ctx.max_query_len * group <= 16
    bound = getattr(ctx, "max_seq_len_bound", 0) or ctx.max_seq_len
    if split_mode and use_tma and tma_decode_supported(qkv.dtype, head_dim, page_size):
        sms = sm_count(qkv.device)
        splits = num_splits or decode_splits_tma(ctx.num_reqs, num_kv_heads, bound, sms)
        scratch = None
        if splits > 1:
            scratch = torch.empty(ctx.num_reqs * num_kv_heads * splits * 16 * (head_dim + 2),
                                  dtype=torch.float32, device=qkv.device)
        k_map, v_map = _kv_tensor_map_pair(k_cache, v_cache)
        _call("kvb_flash_decode_tma", out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0),
              ctypes.addressof(k_map), ctypes.addressof(v_map), table.data_ptr(), table.stride(0),
              ctx.query_start.data_ptr(), ctx.context_lens.data_ptr(), ctx.num_reqs, ctx.max_query_len,
              num_heads, num_kv_heads, head_dim, page_size, num_pages, scale, window,
              splits, None if scratch is None else scratch.data_ptr(),
              None if cos_sin is None else cos_sin.data_ptr(),
              k_cache.data_ptr() if write_kv else None, v_cache.data_ptr() if write_kv else None,
              _decode_work(qkv.device).data_ptr() if TMA_DECODE_SHARED_WORK else None,
              sms * TMA_DECODE_BLOCKS_PER_SM, _stream(),
              kernels=2 if splits > 1 else 1)   # the splits are merged by a second kernel
        return
    if (not split_mode and use_tc5 and tc5_prefill_supported(qkv.dtype, head_dim, page_size)
            and out.stride(0) % 8 == 0):
        k_map, v_map = _kv_tensor_map_pair(k_cache, v_cache, "half")
        _call("kvb_flash_prefill_tc5", out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0),
              ctypes.addressof(k_map), ctypes.addressof(v_map), table.data_ptr(), table.stride(0),
              ctx.query_start.data_ptr(), ctx.context_lens.data_ptr(), ctx.num_reqs, ctx.max_query_len,
              qkv.shape[0], num_heads, num_kv_heads, head_dim, page_size, num_pages, scale, window,
              _stream())
        return
    splits = 1
    if split_mode:
        splits = num_splits or decode_splits(ctx.num_reqs, num_kv_heads, bound, sm_count(qkv.device))
    scratch = None
    if splits > 1:
        scratch = torch.empty(ctx.num_reqs * num_kv_heads * splits * 16 * (head_dim + 2),
                              dtype=torch.float32, device=qkv.device)
    _call("kvb_flash_paged_attention", out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0),
          k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr(), table.stride(0),
          ctx.query_start.data_ptr(), ctx.context_lens.data_ptr(), ctx.num_reqs, ctx.max_query_len,
          num_heads, num_kv_heads, head_dim, page_size, num_pages, scale, window,
          splits, None if scratch is None else scratch.data_ptr(), _stream(), kernels=2 if splits > 1 else 1)


_mm_out_dtype_ok: bool | None = None
# bf16 layers of at most STREAM_AUTO_ROWS tokens (K a multiple of 64) go to this library's own
# weight-streaming kernel (in a whole decode step it measured level with the library product on
# B200 at Llama 3.1 8B shapes, ahead at batch 1); larger batches go to the library product.
# KVCORE_B200_STREAM_ROWS overrides the bound (0: never).
STREAM_MAX_ROWS = 16
STREAM_AUTO_ROWS = int(os.environ.get("KVCORE_B200_STREAM_ROWS", "16"))
_stream_scratch: dict[int, torch.Tensor] = {}


TRACE_TAGS = {1: "gather_rows", 2: "rmsnorm", 3: "silu_mul", 4: "rope_table", 5: "rope_kv_write", 6: "attention_rows",
              7: "flash_paged", 8: "flash_combine", 9: "flash_decode_tma", 10: "flash_decode_combine",
              11: "flash_prefill_tc5", 12: "gemm_f32", 13: "gemm_stream", 14: "sample", 16: "feed_tokens"}
_TRACE_UNITS = ("elementwise", "attention_decode_tma", "attention_flash", "attention_generic",
                "attention_prefill_tc5", "gemm_f32", "sampling", "gemm_stream")
_trace_buffer: torch.Tensor | None = None


def _trace_set(pointer: int | None) -> None:
    for unit in _TRACE_UNITS:
        fn = getattr(_lib, f"kvb_trace_set_{unit}")
        fn.argtypes = [_vp]
        fn.restype = _int
        if fn(pointer) != 0:
            raise KernelError(f"kvb_trace_set_{unit} failed")


def trace_start(device: torch.device | str = "cuda:0", capacity: int = 1 << 16, every_block: bool = False) -> None:
    """Start the kernel timeline trace: the first and last block of every kernel of this library
    (``every_block``: all of them) record when they entered, when the kernel in front had finished,
    and when they left."""
    global _trace_buffer
    ensure_built()
    torch.cuda.synchronize(device)
    buffer = torch.zeros(2 + 4 * capacity, dtype=torch.int64, device=device)
    buffer[1] = capacity | (-(1 << 63) if every_block else 0)
    with torch.cuda.device(device):
        _trace_set(buffer.data_ptr())
    _trace_buffer = buffer


def trace_stop() -> list[dict]:
    """Stop the trace; events sorted by entry time: kernel, block ("first"/"last"/"other"), sm, index
    (linear block index), entry, waited, exit (ns)."""
    global _trace_buffer
    if _trace_buffer is None:
        return []
    buffer = _trace_buffer
    torch.cuda.synchronize(buffer.device)
    with torch.cuda.device(buffer.device):
        _trace_set(None)
    host = buffer.cpu().tolist()
    _trace_buffer = None
    count = min(host[0], host[1] & ((1 << 63) - 1))
    events = []
    for i in range(count):
        tag, entry, waited, leave = host[2 + 4 * i: 6 + 4 * i]
        events.append({"kernel": TRACE_TAGS.get(tag & 0xFF, str(tag & 0xFF)),
                       "block": ("first", "last", "other")[min((tag >> 8) & 3, 2)], "sm": (tag >> 12) & 0x3FF,
                       "index": (tag >> 32) & 0xFFFFFFFF, "entry": entry, "waited": waited, "exit": leave})
    events.sort(key=lambda e: e["entry"])
    return events


def set_overlapped_launch(enabled: bool) -> None:
    """Switch programmatic dependent launch on or off for this library's kernels."""
    ensure_built()
    _lib.kvb_set_pdl(1 if enabled else 0)


def linear_stream(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, *,
                  out_dtype: torch.dtype | None = None, silu_pairs: bool = False) -> torch.Tensor:
    """``x @ weight.T`` for a decode-sized batch of bf16 ``x`` (at most 16 rows), K a multiple of 64: a
    balanced weight-streaming kernel (one block per SM, every block the same number of bytes).

    ``silu_pairs``: the rows of ``weight`` alternate in runs of 8 gate rows and 8 up rows; the
    result is ``[M, N/2]``, ``silu(gate) * up``, with the roundings of the unfused path."""
    _check(x, "x", dtype=torch.bfloat16, contiguous=False)
    _check(weight, "weight", dtype=torch.bfloat16)
    m, k = x.shape
    n = weight.shape[0]
    if not 0 < m <= STREAM_MAX_ROWS or k % 64 or x.stride(1) != 1 or x.stride(0) % 8:
        raise KernelError(f"linear_stream: unsupported shape x {tuple(x.shape)} strides {x.stride()}")
    if bias is not None:
        _check(bias, "bias", dtype=torch.bfloat16)
    if silu_pairs and (n % 16 or out_dtype not in (None, torch.bfloat16)):
        raise KernelError("linear_stream: gated pairs need an output width that is a multiple of 16 and a bf16 result")
    out = torch.empty((m, n // 2 if silu_pairs else n), dtype=out_dtype or torch.bfloat16, device=x.device)
    _stream_call(x.device, out.data_ptr(), int(out.dtype == torch.float32), out.stride(0),
                 x.data_ptr(), x.stride(0), weight.data_ptr(), None if bias is None else bias.data_ptr(),
                 m, n, k, int(silu_pairs), None, 0, 0.0, None, 0, None, None)
    return out


def linear(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None = None,
    *,
    out_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` for ``x [M, K]``, ``weight [N, K]``.

    float32: this package's own FMA kernel (no tensor cores, fixed summation order).
    bfloat16: the library matrix product with 32-bit accumulation.
    ``out_dtype=float32`` keeps the accumulator's precision in the result (the logits).
    """
    global _mm_out_dtype_ok
    _check(x, "x", contiguous=False)
    _check(weight, "weight", dtype=x.dtype)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise KernelError(f"linear: x {tuple(x.shape)} does not match weight {tuple(weight.shape)}")
    if x.stride(1) != 1:
        x = x.contiguous()
    m, k = x.shape
    n = weight.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        _call("kvb_gemm_f32", out.data_ptr(), x.data_ptr(), weight.data_ptr(),
              None if bias is None else bias.data_ptr(), m, n, k, x.stride(0), out.stride(0), _stream())
        return out
    # Decode-sized batches: the layer is one pass over the weights, which this library's own
    # streaming kernel does, overlapping its start with the kernels in front of it.
    if _stream_ok(x, weight):
        return linear_stream(x, weight, bias, out_dtype=out_dtype)
    if out_dtype == torch.float32:
        if _mm_out_dtype_ok is None:
            try:
                torch.mm(x[:1], weight[:1].t(), out_dtype=torch.float32)
                _mm_out_dtype_ok = True
            except (TypeError, RuntimeError):
                _mm_out_dtype_ok = False
        if _mm_out_dtype_ok:
            out = torch.mm(x, weight.t(), out_dtype=torch.float32)
        else:
            out = torch.mm(x, weight.t()).float()
        if bias is not None:
            out = out + bias.float()
        return out
    return torch.nn.functional.linear(x, weight, bias)


def _stream_buffers(device: torch.device) -> torch.Tensor:
    """Scratch of the streaming kernel; kept for good, since a captured graph holds its address.  Every
    word holds a marker between launches."""
    index = device.index or 0
    scratch = _stream_scratch.get(index)
    if scratch is None:
        floats = int(_lib.kvb_gemm_stream_scratch_floats(sm_count(device)))
        marker = int(_lib.kvb_gemm_stream_scratch_marker())
        words = torch.full((floats,), marker, dtype=torch.int32, device=device)
        scratch = _stream_scratch[index] = words.view(torch.float32)
    return scratch


def _stream_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the streaming kernel takes ``x @ weight.T`` (at most STREAM_AUTO_ROWS tokens); otherwise
    the library product does.  A streaming kernel on tcgen05 for 17 to 128 tokens existed and was
    taken out: in whole decode steps at Llama 3.1 8B layer sizes it was 29 % slower than the library
    product at 20 and 32 tokens and 39 to 47 % slower at 48 and 64."""
    m, k = x.shape
    return (x.dtype == torch.bfloat16 and k % 64 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and 0 < m <= min(STREAM_AUTO_ROWS, STREAM_MAX_ROWS))


_STREAM_PIECE = 64   # columns of the residual whose squares one piece of ``sumsq`` holds


def _stream_call(device: torch.device, *args) -> None:
    """``kvb_gemm_stream_bf16`` with ``args`` up to ``sumsq_out``; scratch, SM count and stream are appended."""
    _call("kvb_gemm_stream_bf16", *args, _stream_buffers(device).data_ptr(), sm_count(device), _stream())


def linear_silu_mul(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, *,
                    group: int = 0) -> torch.Tensor:
    """The first half of a gated feed-forward: ``silu(gate(x)) * up(x)`` for a packed ``[2I, E]``
    matrix whose gate and up rows are halves (``group == 0``) or alternate in runs of ``group``.
    Decode-sized bf16 batches with runs of 8 take the streaming kernel with the activation in
    its epilogue; everything else is the matrix product followed by ``silu_mul``."""
    _check(x, "x", contiguous=False)
    _check(weight, "weight", dtype=x.dtype)
    if group == 8 and x.dim() == 2 and _stream_ok(x, weight) and weight.shape[0] % 16 == 0:
        return linear_stream(x, weight, bias, silu_pairs=True)
    return silu_mul(linear(x, weight, bias), group)


def norm_linear(h: torch.Tensor | None, residual: torch.Tensor | None, norm_weight: torch.Tensor, eps: float,
                weight: torch.Tensor, bias: torch.Tensor | None = None, *, silu_group: int | None = None,
                sumsq: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """A sub-layer's entry: ``x = rmsnorm(h + residual)``, then ``x @ weight.T`` (``silu_group`` None)
    or the gated ``silu(gate(x)) * up(x)`` (``silu_group`` as in ``linear_silu_mul``).

    Returns ``(out, residual)`` with ``residual`` now holding the sum (``residual`` None: the sum is
    ``h`` itself).  ``h`` None means the sub-layer in front has already added its output into
    ``residual`` (see ``linear_add_residual``); if it also left the rows' squares in ``sumsq``, a
    decode-sized bf16 batch runs as ONE kernel: a warp of the streaming product scales each stage's
    token rows by ``norm_weight * rsqrt(mean + eps)`` before they are used.  Everything else is
    the norm kernel followed by the product."""
    if h is None:
        if residual is None:
            raise KernelError("norm_linear: nothing to normalise")
        _check(residual, "residual", contiguous=False)
        m, k = residual.shape
        weight_bytes = 4 if norm_weight.dtype == torch.float32 else 2
        if (sumsq is not None and _stream_ok(residual, weight)
                and k * weight_bytes <= 4 * int(_lib.kvb_gemm_stream_norm_max_k())
                and norm_weight.dtype in (torch.bfloat16, torch.float32) and norm_weight.is_contiguous()
                and norm_weight.data_ptr() % 16 == 0
                and sumsq.dtype == torch.float32 and sumsq.is_contiguous() and sumsq.shape[0] == m
                and (silu_group is None or (silu_group == 8 and weight.shape[0] % 16 == 0))):
            _check(weight, "weight", dtype=torch.bfloat16)
            if bias is not None:
                _check(bias, "bias", dtype=torch.bfloat16)
            n = weight.shape[0]
            out = torch.empty((m, n // 2 if silu_group else n), dtype=torch.bfloat16, device=residual.device)
            _stream_call(residual.device, out.data_ptr(), 0, out.stride(0), residual.data_ptr(),
                         residual.stride(0), weight.data_ptr(), None if bias is None else bias.data_ptr(), m, n, k,
                         int(bool(silu_group)), norm_weight.data_ptr(), int(norm_weight.dtype == torch.float32),
                         float(eps), sumsq.data_ptr(), sumsq.shape[1], None, None)
            return out, residual
        x = rmsnorm(residual, norm_weight, eps)
    elif residual is None:
        x, residual = rmsnorm(h, norm_weight, eps), h
    else:
        x = add_rmsnorm(h, residual, norm_weight, eps)
    out = linear(x, weight, bias) if silu_group is None else linear_silu_mul(x, weight, bias, group=silu_group)
    return out, residual


def linear_add_residual(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                        residual: torch.Tensor | None) -> tuple[torch.Tensor | None, torch.Tensor | None]:
    """A sub-layer's exit: ``out = x @ weight.T (+ bias)`` on its way into the residual stream.

    Decode-sized bf16 batches: the streaming product adds its (bf16-rounded) result into ``residual``
    in place and returns ``(None, sumsq)``, ``sumsq [T, ceil(N / 64)]`` being the squares of the new
    rows of ``residual``, 64 columns a piece, for the norm that follows.  Otherwise returns
    ``(out, None)``: the sum is left to that norm, as the deferred-residual scheme has it."""
    if (residual is not None and x.dim() == 2 and _stream_ok(x, weight)
            and weight.shape[0] % 8 == 0 and residual.dtype == torch.bfloat16 and residual.is_contiguous()
            and tuple(residual.shape) == (x.shape[0], weight.shape[0]) and residual.data_ptr() % 16 == 0):
        _check(weight, "weight", dtype=torch.bfloat16)
        if bias is not None:
            _check(bias, "bias", dtype=torch.bfloat16)
        m, k = x.shape
        n = weight.shape[0]
        sumsq = torch.empty((m, -(-n // _STREAM_PIECE)), dtype=torch.float32, device=x.device)
        _stream_call(x.device, None, 0, n, x.data_ptr(), x.stride(0), weight.data_ptr(),
                     None if bias is None else bias.data_ptr(), m, n, k, 0, None, 0, 0.0, None, 0,
                     residual.data_ptr(), sumsq.data_ptr())
        return None, sumsq
    return linear(x, weight, bias), None


def sample(logits: torch.Tensor, packed_params: torch.Tensor, eps: float) -> torch.Tensor:
    """One token per row of ``logits [S, V]`` float32; ``packed_params [S, 6]`` float64 (on the
    device already, or on the host: then copied): temperature, top_k, top_p, seed low 32 bits, seed
    high 32 bits, index of the sampled token."""
    _check(logits, "logits", dtype=torch.float32)
    rows, vocab = logits.shape
    params = packed_params.to(device=logits.device, dtype=torch.float64, non_blocking=False).contiguous()
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _call("kvb_sample", out.data_ptr(), logits.data_ptr(), params.data_ptr(), rows, vocab, float(eps), _stream())
    return out


__all__ = [
    "KernelError",
    "add_rmsnorm",
    "check_attention_shape",
    "ensure_built",
    "feed_tokens",
    "decode_splits",
    "decode_splits_tma",
    "flash_attention_supported",
    "tc5_prefill_supported",
    "tma_decode_supported",
    "gather_rows",
    "library_is_loaded",
    "linear",
    "linear_add_residual",
    "linear_silu_mul",
    "linear_stream",
    "norm_linear",
    "set_overlapped_launch",
    "sm_count",
    "trace_start",
    "trace_stop",
    "paged_attention",
    "read_status",
    "peek_status",
    "raise_on_status",
    "require_device",
    "rmsnorm",
    "rope_inplace",
    "rope_kv_write",
    "rope_table",
    "sample",
    "silu_mul",
]
