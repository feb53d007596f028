"""Bind checkpoint tensors to a model's weight slots by name, with one collected error.

The reference binds by name through a rename table and copies into stacked parameters
(kvcore/model/model_utils.py:37-128; kvcore/model/models/llama3.py:249-262), ignores unknown
names, and reports only missing ones (default_loader.py:179-196).  Here every part declares
its own slots (a slot may be a row range of a packed matrix), and the loader reports missing
tensors, unexpected tensors and wrong shapes together in a single ``WeightLoadError``.

Precision: floating tensors are cast to the slot's dtype (the model's compute dtype);
integer tensors are kept as int32; a slot marked ``keep_f32`` whose tensor the file stores
in 32-bit keeps it in 32-bit even in a bfloat16 model.
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterable, Mapping

import torch

from ..parts.base import WeightSlot
from .safetensors_io import SafetensorsFile, weight_files


class WeightLoadError(ValueError):
    """Lists every missing tensor, unexpected tensor and shape mismatch of a load."""

    def __init__(
        self,
        missing: list[str],
        unexpected: list[str],
        wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]],
        source: str = "",
    ) -> None:
        self.missing = missing
        self.unexpected = unexpected
        self.wrong_shape = wrong_shape
        lines = [f"weights{' in ' + source if source else ''} do not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            parts = [f"{name}: file {list(got)} vs model {list(want)}" for name, got, want in wrong_shape]
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(parts))
        super().__init__("\n".join(lines))


def _copy_into(slot: WeightSlot, tensor: torch.Tensor) -> None:
    dest = slot.dest
    if tuple(tensor.shape) != tuple(dest.shape):   # a scattering view: same elements, same order
        tensor = tensor.reshape(dest.shape)
    if (
        slot.keep_f32
        and slot.rebind is not None
        and tensor.dtype == torch.float32
        and dest.dtype != torch.float32
    ):
        slot.rebind(tensor.to(device=dest.device, dtype=torch.float32).contiguous())
        return
    if not tensor.dtype.is_floating_point and dest.dtype == torch.int32:
        dest.copy_(tensor.to(torch.int32))
        return
    dest.copy_(tensor.to(device=dest.device, dtype=dest.dtype, non_blocking=False))


def load_named_tensors(
    slots: Iterable[WeightSlot],
    tensors: Iterable[tuple[str, torch.Tensor]],
    *,
    ignorable: Iterable[str] = (),
    strict: bool = True,
    source: str = "",
) -> set[str]:
    """Copy ``tensors`` into ``slots`` by name; return the names loaded.

    ``ignorable`` names may be present in the checkpoint without a slot; the parts name them
    (a tied output matrix, a frequency table that a part derives itself).  With ``strict`` any mismatch raises after all
    tensors were looked at, so the message is complete.
    """
    by_name: dict[str, WeightSlot] = {}
    for slot in slots:
        if slot.name in by_name:
            raise ValueError(f"two weight slots share the name {slot.name!r}")
        by_name[slot.name] = slot
    ignorable = set(ignorable)
    loaded: set[str] = set()
    unexpected: list[str] = []
    wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]] = []
    for name, tensor in tensors:
        slot = by_name.get(name)
        if slot is None:
            if name not in ignorable:
                unexpected.append(name)
            continue
        if tuple(tensor.shape) != slot.shape:
            wrong_shape.append((name, tuple(tensor.shape), slot.shape))
            continue
        _copy_into(slot, tensor)
        loaded.add(name)
    missing = [name for name in by_name if name not in loaded and name not in {w[0] for w in wrong_shape}]
    if strict and (missing or unexpected or wrong_shape):
        raise WeightLoadError(sorted(missing), sorted(unexpected), wrong_shape, source)
    return loaded


def iterate_folder(folder: str | Path) -> Iterable[tuple[str, torch.Tensor]]:
    for path in weight_files(folder):
        with SafetensorsFile(path) as handle:
            for name in handle.names():
                yield name, handle.tensor(name)


def load_model_weights(model, folder: str | Path, *, strict: bool = True) -> set[str]:
    """Fill ``model`` (anything with ``weight_slots()``, ``ignorable_tensor_names()`` and
    ``finalize_weights()``) from the safetensors files of ``folder``."""
    loaded = load_named_tensors(
        model.weight_slots(),
        iterate_folder(folder),
        ignorable=model.ignorable_tensor_names(),
        strict=strict,
        source=str(folder),
    )
    model.finalize_weights()
    return loaded


def load_state_dict(model, tensors: Mapping[str, torch.Tensor], *, strict: bool = True) -> set[str]:
    """Same as ``load_model_weights`` from an in-memory mapping of checkpoint names."""
    loaded = load_named_tensors(
        model.weight_slots(),
        tensors.items(),
        ignorable=model.ignorable_tensor_names(),
        strict=strict,
        source="state dict",
    )
    model.finalize_weights()
    return loaded


__all__ = [
    "WeightLoadError",
    "iterate_folder",
    "load_model_weights",
    "load_named_tensors",
    "load_state_dict",
]
