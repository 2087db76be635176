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
import os
import struct
from ctypes import POINTER, byref, c_char_p, c_int, c_longlong, c_ubyte, c_void_p

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


_lib = None


def _runtime():
    global _lib
    if _lib is None:
        from ..kernels import build
        lib = build.load("host_runtime")
        lib.ri_st_open.restype = c_void_p
        lib.ri_st_open.argtypes = [c_char_p]
        lib.ri_st_close.restype = None
        lib.ri_st_close.argtypes = [c_void_p]
        lib.ri_st_count.argtypes = [c_void_p]
        lib.ri_st_entry.argtypes = [c_void_p, c_int, POINTER(c_char_p), POINTER(c_char_p), POINTER(c_int),
                                    POINTER(POINTER(c_longlong)), POINTER(c_longlong), POINTER(c_longlong)]
        lib.ri_st_data.restype = c_void_p
        lib.ri_st_data.argtypes = [c_void_p, POINTER(c_longlong)]
        lib.ri_st_metadata_count.argtypes = [c_void_p]
        lib.ri_st_metadata.argtypes = [c_void_p, c_int, POINTER(c_char_p), POINTER(c_char_p)]
        _lib = lib
    return _lib


class SafetensorsFile:
    """A memory-mapped safetensors file; `tensor(name)` copies nothing until asked.  The native host
    runtime (`csrc/host_runtime.cpp`) opens and maps the file and reads and checks its header."""

    def __init__(self, path: str):
        self.path = path
        self._rt = _runtime()
        self._h = c_void_p(self._rt.ri_st_open(os.fsencode(path)))
        if not self._h:
            raise WeightFileError(self._rt.ri_last_error().decode("utf-8", "replace"))
        try:
            self.metadata = {}
            key, value = c_char_p(), c_char_p()
            for i in range(self._rt.ri_st_metadata_count(self._h)):
                self._rt.ri_st_metadata(self._h, i, byref(key), byref(value))
                self.metadata[key.value.decode("utf-8")] = value.value.decode("utf-8")
            self.entries: dict[str, dict] = {}
            name, dtype, ndim = c_char_p(), c_char_p(), c_int()
            shape, begin, end = POINTER(c_longlong)(), c_longlong(), c_longlong()
            for i in range(self._rt.ri_st_count(self._h)):
                self._rt.ri_st_entry(self._h, i, byref(name), byref(dtype), byref(ndim), byref(shape), byref(begin),
                                     byref(end))
                self.entries[name.value.decode("utf-8")] = {
                    "dtype": dtype.value.decode("utf-8"), "shape": tuple(int(shape[k]) for k in range(ndim.value)),
                    "begin": begin.value, "end": end.value}
        except UnicodeDecodeError:
            self.close()
            raise WeightFileError(f"{path}: header is not valid JSON: a name is not UTF-8") from None
        length = c_longlong()
        self._data = self._rt.ri_st_data(self._h, byref(length))

    def names(self):
        return list(self.entries)

    def shape(self, name: str) -> tuple:
        return self.entries[name]["shape"]

    def dtype_name(self, name: str) -> str:
        return self.entries[name]["dtype"]

    def supported(self, name: str) -> bool:
        return self.entries[name]["dtype"] in _DTYPES

    def tensor(self, name: str) -> torch.Tensor:
        if not self._h:
            raise WeightFileError(f"{self.path}: the file has been closed")
        e = self.entries[name]
        if e["dtype"] not in _DTYPES:
            raise WeightFileError(f"{self.path}: {name!r} has unsupported dtype {e['dtype']}")
        dtype, _ = _DTYPES[e["dtype"]]
        n_bytes = e["end"] - e["begin"]
        if n_bytes:
            mapped = np.ctypeslib.as_array((c_ubyte * n_bytes).from_address(self._data + e["begin"]))
            t = torch.from_numpy(mapped.copy())    # one tensor at a time leaves the map
        else:
            t = torch.empty(0, dtype=torch.uint8)
        t = t.view(dtype).reshape(e["shape"])
        if dtype == torch.float16:
            t = t.to(torch.float32)
        elif dtype == torch.int64:
            t = t.to(torch.int32)
        return t

    def close(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._rt.ri_st_close(h)

    def __del__(self):
        try:
            self.close()
        except Exception:              # the interpreter is shutting down and the library is gone
            pass


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
