"""Reading and writing the safetensors container, without any model knowledge.

Format (as the reference parses it, src/model/safetensors_loader.cpp:469-568):
an 8-byte little-endian header length, a JSON object that maps each tensor name
to {"dtype", "shape", "data_offsets": [begin, end]} relative to the end of the
header (plus an optional "__metadata__" entry), then the raw little-endian data.
A folder may also hold `model.safetensors.index.json` naming several shard files.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are views of the mapping."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (only {size} bytes)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        data_size = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dt, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}'") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            tdt, isz = _DTYPES[dt]
            if b < 0 or en < b or en > data_size:
                raise SafetensorsError(f"{path}: tensor '{name}' data range [{b},{en}) lies outside the "
                                       f"file's data section of {data_size} bytes (truncated file?)")
            if en - b != _numel(shape) * isz:
                raise SafetensorsError(f"{path}: tensor '{name}' has {en - b} bytes but shape {list(shape)} "
                                       f"of {dt} needs {_numel(shape) * isz}")
            self.entries[name] = (tdt, shape, b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self):
        return list(self.entries)

    def info(self, name: str):
        dt, shape, _, _ = self.entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor's bytes in the mapping (copy before writing)."""
        dt, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        buf = memoryview(self._mm)[self._data_start + b:self._data_start + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # non-writable buffer: the view is never written
            t = torch.frombuffer(buf, dtype=dt)
        return t.reshape(shape)

    def close(self):
        # Views handed out keep the mapping alive; only the descriptor is dropped here.
        try:
            self._f.close()
        except Exception:
            pass


def open_model_files(model_dir: str):
    """All safetensors files of a model folder: [SafetensorsFile].

    A single `model.safetensors`, or the shards named by
    `model.safetensors.index.json`'s weight_map.
    """
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            wm = json.load(f).get("weight_map", {})
        shard_names = sorted(set(wm.values()))
        missing = [s for s in shard_names if not os.path.exists(os.path.join(model_dir, s))]
        if missing:
            raise SafetensorsError(f"{index}: shard files missing: {missing}")
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shard_names]
    if os.path.exists(single):
        return [SafetensorsFile(single)]
    raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in {model_dir}")


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write `tensors` (CPU or device; made contiguous) as one safetensors file."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - (len(hjson) % 8)) % 8
    hjson += b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel() == 0:
                continue
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
