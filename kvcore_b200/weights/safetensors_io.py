"""Minimal safetensors reader and writer (no third-party dependency).

File layout: 8 bytes little-endian header length N, N bytes of JSON mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end
of the header), then the raw little-endian tensor bytes.  The reference reads the same
files through the safetensors package (kvcore/model/model_loader/weight_utils.py:11-19).
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Iterator, Mapping

import torch

_DTYPES: dict[str, torch.dtype] = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_DTYPE_NAMES = {dtype: name for name, dtype in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors file."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """Read-only, memory-mapped view of one .safetensors file."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        self._handle = self.path.open("rb")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too small to be a safetensors file")
        (header_len,) = struct.unpack("<Q", self._handle.read(8))
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(f"{self.path}: header length {header_len} exceeds the file size")
        try:
            header = json.loads(self._handle.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({exc})") from exc
        self._data_start = 8 + header_len
        self.metadata: Mapping[str, str] = header.pop("__metadata__", {}) or {}
        self.entries: dict[str, TensorEntry] = {}
        data_len = size - self._data_start
        for name, info in header.items():
            dtype_name = info.get("dtype")
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {dtype_name!r}")
            begin, end = info["data_offsets"]
            shape = tuple(int(x) for x in info["shape"])
            numel = 1
            for extent in shape:
                numel *= extent
            expected = numel * _DTYPES[dtype_name].itemsize
            if begin < 0 or end > data_len or end - begin != expected:
                raise SafetensorsError(
                    f"{self.path}: tensor {name!r} has data_offsets [{begin}, {end}) that do not "
                    f"match shape {list(shape)} of {dtype_name}"
                )
            self.entries[name] = TensorEntry(name, _DTYPES[dtype_name], shape, begin, end)
        self._mmap = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> list[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor as a CPU tensor sharing the mapped file's memory (do not write to it)."""
        entry = self.entries[name]
        numel = 1
        for extent in entry.shape:
            numel *= extent
        if numel == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the read-only buffer warning: callers copy, never write
            flat = torch.frombuffer(
                self._mmap, dtype=entry.dtype, count=numel, offset=self._data_start + entry.begin
            )
        return flat.view(entry.shape)

    def items(self) -> Iterator[tuple[str, torch.Tensor]]:
        for name in self.entries:
            yield name, self.tensor(name)

    def close(self) -> None:
        if self._mmap is not None:
            try:
                self._mmap.close()
            except BufferError:
                pass  # tensors still view the mapping; it is released with them
            self._mmap = None
        self._handle.close()

    def __enter__(self) -> "SafetensorsFile":
        return self

    def __exit__(self, *exc_info: object) -> None:
        self.close()


def write_safetensors(
    path: str | Path,
    tensors: Mapping[str, torch.Tensor],
    metadata: Mapping[str, str] | None = None,
) -> None:
    """Write tensors (any device; moved to CPU) to ``path`` in name order."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    ordered = sorted(tensors)
    for name in ordered:
        tensor = tensors[name]
        if tensor.dtype not in _DTYPE_NAMES:
            raise SafetensorsError(f"tensor {name!r} has dtype {tensor.dtype} that safetensors cannot hold")
        nbytes = tensor.numel() * tensor.dtype.itemsize
        header[name] = {
            "dtype": _DTYPE_NAMES[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)  # keep tensor data 8-byte aligned
    with Path(path).open("wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name in ordered:
            tensor = tensors[name].detach().contiguous().cpu()
            handle.write(tensor.view(torch.uint8).numpy().tobytes() if tensor.numel() else b"")


def weight_files(folder: str | Path) -> list[Path]:
    """The safetensors files of a model folder: those the index names, else all of them.

    Same resolution order as the reference (default_loader.py:98-128; weight_utils.py:38-52).
    """
    folder = Path(folder)
    if not folder.is_dir():
        raise FileNotFoundError(f"model folder {str(folder)!r} does not exist")
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        with index.open("r", encoding="utf-8") as handle:
            weight_map = json.load(handle).get("weight_map", {})
        files = sorted({folder / name for name in weight_map.values()})
    else:
        files = sorted(folder.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"cannot find any .safetensors weights in {str(folder)!r}")
    return files


__all__ = ["SafetensorsError", "SafetensorsFile", "TensorEntry", "weight_files", "write_safetensors"]
