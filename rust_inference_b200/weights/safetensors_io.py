"""Reading and writing safetensors files, by tensor name.

Format: an 8-byte little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}}` and the raw little-endian
data.  The role is the one gguf.rs plays in the reference (name -> type, shape, bytes;
errors on a bad header: gguf.rs:255-341); the format itself is the model folder's.

Tensors come back in the precision they were stored in: BF16 stays bfloat16, F32 stays
float32, F16 is widened to float32 (exact), integer tensors become int32.
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import numpy as np
import torch


class WeightFileError(ValueError):
    """The file is not a readable safetensors file."""


_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
          torch.int32: "I32", torch.int64: "I64"}


class SafetensorsFile:
    """A memory-mapped safetensors file; `tensor(name)` copies nothing until asked."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError as e:
            raise WeightFileError(f"{path}: {e.strerror}") from None
        if size < 8:
            raise WeightFileError(f"{path}: too short to hold a safetensors header")
        self._file = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._file.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise WeightFileError(f"{path}: header length {hlen} does not fit a file of {size} bytes")
        try:
            header = json.loads(self._file.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise WeightFileError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: dict[str, dict] = {}
        for name, e in header.items():
            try:
                dtype, shape, (begin, end) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise WeightFileError(f"{path}: malformed header entry for {name!r}") from None
            if dtype in _DTYPES:
                want = _DTYPES[dtype][1] * int(np.prod(shape, dtype=np.int64)) if shape else _DTYPES[dtype][1]
                if end - begin != want:
                    raise WeightFileError(
                        f"{path}: {name!r} has {end - begin} bytes, shape {list(shape)} of {dtype} needs {want}")
            if begin < 0 or end < begin or end > data_len:
                raise WeightFileError(
                    f"{path}: {name!r} data_offsets [{begin}, {end}) lie outside the {data_len} data bytes")
            self.entries[name] = {"dtype": dtype, "shape": shape, "begin": begin, "end": end}
        self._mmap = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self):
        return list(self.entries)

    def shape(self, name: str) -> tuple:
        return self.entries[name]["shape"]

    def dtype_name(self, name: str) -> str:
        return self.entries[name]["dtype"]

    def supported(self, name: str) -> bool:
        return self.entries[name]["dtype"] in _DTYPES

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e["dtype"] not in _DTYPES:
            raise WeightFileError(f"{self.path}: {name!r} has unsupported dtype {e['dtype']}")
        dtype, _ = _DTYPES[e["dtype"]]
        n_bytes = e["end"] - e["begin"]
        raw = np.frombuffer(self._mmap, dtype=np.uint8, count=n_bytes, offset=self._data_start + e["begin"])
        t = torch.from_numpy(raw.copy())       # one tensor at a time leaves the map
        t = t.view(dtype).reshape(e["shape"])
        if dtype == torch.float16:
            t = t.to(torch.float32)
        elif dtype == torch.int64:
            t = t.to(torch.int32)
        return t

    def close(self):
        if self._mmap is not None:
            self._mmap.close()
            self._mmap = None
        self._file.close()


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Write tensors (CPU or device; float32, bfloat16, float16, int32, int64) to one file."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightFileError(f"cannot store {name!r} of dtype {t.dtype}")
        n_bytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + n_bytes]}
        offset += n_bytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-(8 + len(blob)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


class ModelFiles:
    """All safetensors files of a model folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` (`weight_map`) names."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self.files: list[SafetensorsFile] = []
        self.where: dict[str, SafetensorsFile] = {}
        if os.path.isfile(single):
            paths = [single]
        elif os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                try:
                    weight_map = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise WeightFileError(f"{index}: no readable 'weight_map'") from None
            paths = [os.path.join(model_dir, p) for p in sorted(set(weight_map.values()))]
        else:
            raise WeightFileError(f"no model.safetensors (or index) in model folder {model_dir!r}")
        for p in paths:
            sf = SafetensorsFile(p)
            self.files.append(sf)
            for name in sf.names():
                self.where[name] = sf

    def names(self):
        return list(self.where)

    def shape(self, name):
        return self.where[name].shape(name)

    def dtype_name(self, name):
        return self.where[name].dtype_name(name)

    def supported(self, name):
        return self.where[name].supported(name)

    def tensor(self, name):
        return self.where[name].tensor(name)

    def close(self):
        for f in self.files:
            f.close()
