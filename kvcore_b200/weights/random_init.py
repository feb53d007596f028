"""Seeded random weights: fill a model in place, or write a model folder from a configuration.

The reference has no such mode; its tests build modules under ``torch.manual_seed`` with
torch's default initialisers (tests/test_model_loading.py:146-148).  Here every tensor whose
slot says "normal" is drawn from N(0, std) in 32-bit and then cast, "ones" and "zeros" are
filled; tensors are visited in sorted name order so the stream of one seed is fixed.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

import torch

from ..config.engine_config import normalize_dtype_name
from ..config.registry import model_spec_from_config
from .safetensors_io import write_safetensors

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _fill(dest: torch.Tensor, init: str, std: float, generator: torch.Generator) -> None:
    if init == "ones":
        dest.fill_(1.0)
    elif init == "zeros":
        dest.zero_()
    elif init == "normal":
        # draw in 32-bit, then round: a bfloat16 and a float32 model of one seed share values
        rows = dest.shape[0] if dest.dim() > 1 else 1
        step = max(1, (1 << 26) // max(1, dest.numel() // rows))
        if dest.dim() <= 1:
            values = torch.empty(dest.shape, dtype=torch.float32, device=generator.device)
            values.normal_(0.0, std, generator=generator)
            dest.copy_(values)
            return
        for begin in range(0, rows, step):
            chunk = dest[begin : begin + step]
            values = torch.empty(chunk.shape, dtype=torch.float32, device=generator.device)
            values.normal_(0.0, std, generator=generator)
            chunk.copy_(values)
    else:
        raise ValueError(f"unknown weight init {init!r}")


def init_random_weights_(model, seed: int, std: float = 0.02) -> None:
    """Fill every weight slot of ``model`` in place on its own device, then finalize."""
    slots = sorted(model.weight_slots(), key=lambda slot: slot.name)
    if not slots:
        return
    device = slots[0].dest.device
    generator = torch.Generator(device=device)
    generator.manual_seed(int(seed))
    for slot in slots:
        _fill(slot.dest, slot.init, std, generator)
    model.finalize_weights()


def random_state_dict(
    config: Mapping[str, Any], seed: int, std: float = 0.02, dtype: str = "bfloat16"
) -> dict[str, torch.Tensor]:
    """Checkpoint-named CPU tensors for ``config`` (a config.json dict), drawn from ``seed``."""
    from ..parts.model import build_model  # late: parts import this package's loader

    torch_dtype = _TORCH_DTYPES[normalize_dtype_name(dtype)]
    spec = model_spec_from_config(config)
    skeleton = build_model(spec, dtype=torch_dtype, device=torch.device("meta"))
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    tensors: dict[str, torch.Tensor] = {}
    for slot in sorted(skeleton.weight_slots(), key=lambda slot: slot.name):
        dest = torch.empty(slot.shape, dtype=torch_dtype)
        _fill(dest, slot.init, std, generator)
        tensors[slot.name] = dest
    return tensors


def write_random_model(
    folder: str | Path,
    config: Mapping[str, Any],
    seed: int,
    std: float = 0.02,
    dtype: str = "bfloat16",
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a random model of ``config``."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    dtype = normalize_dtype_name(dtype)
    tensors = random_state_dict(config, seed, std, dtype)
    stored = dict(config)
    stored["torch_dtype"] = dtype
    with (folder / "config.json").open("w", encoding="utf-8") as handle:
        json.dump(stored, handle, indent=2, sort_keys=True)
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt", "seed": str(seed)})
    return folder


__all__ = ["init_random_weights_", "random_state_dict", "write_random_model"]
