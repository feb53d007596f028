"""Hand-written sm_100a CUDA kernels and their Python wrappers.

Parts call these through ``kvcore_b200.kernels.<name>`` at call time.
"""
from . import api
from .api import (
    KernelError,
    add_rmsnorm,
    check_attention_shape,
    decode_splits,
    decode_splits_tma,
    tc5_prefill_supported,
    tma_decode_supported,
    ensure_built,
    flash_attention_supported,
    gather_rows,
    library_is_loaded,
    linear,
    linear_skinny,
    paged_attention,
    read_status,
    require_device,
    rmsnorm,
    rope_inplace,
    rope_kv_write,
    rope_table,
    sample,
    silu_mul,
)

__all__ = [
    "KernelError",
    "add_rmsnorm",
    "check_attention_shape",
    "decode_splits",
    "decode_splits_tma",
    "tc5_prefill_supported",
    "tma_decode_supported",
    "ensure_built",
    "flash_attention_supported",
    "gather_rows",
    "library_is_loaded",
    "linear",
    "linear_skinny",
    "paged_attention",
    "read_status",
    "require_device",
    "rmsnorm",
    "rope_inplace",
    "rope_kv_write",
    "rope_table",
    "sample",
    "silu_mul",
]
