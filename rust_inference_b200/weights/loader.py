"""Fetching a model's tensors from its folder by name, and the random-weights mode.

The reference reads every tensor into a map and then takes them out by name, failing
on the first missing one (model.rs:157-203) and never checking a shape against the
config (model.rs:205, :246-249).  Here the model declares every tensor it wants with
its shape; the folder is compared with that declaration as a whole, and ONE error lists
all missing tensors, all unexpected ones, every wrong shape and every unsupported dtype.
"""
from __future__ import annotations

import fnmatch
import json
import os
import warnings
import zlib
from typing import Iterator, Mapping

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import ModelFiles, write_safetensors


class WeightError(ValueError):
    """The folder's tensors do not match what the model declares."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape, bad_dtype):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)      # (name, expected, found)
        self.bad_dtype = list(bad_dtype)          # (name, dtype name)
        lines = [f"weights in {model_dir!r} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name}: expected {list(want)}, found {list(got)}")
        for name, dt in self.bad_dtype:
            lines.append(f"  unsupported dtype: {name}: {dt}")
        super().__init__("\n".join(lines))


def check_tensors(files: ModelFiles, expected: Mapping[str, TensorSpec], ignore=()) -> list:
    """Compare the folder with the declaration; raises ONE `WeightError` for everything that is
    wrong.  `ignore`: name patterns (fnmatch) of tensors a folder may hold although the model does
    not use them (a stored head beside tied embeddings, rotary frequency tables of old exports):
    the reference takes the tensors it needs by name and leaves the rest (model.rs:157-203).  They
    are returned, and the caller warns; every other undeclared tensor stays an error."""
    have = set(files.names())
    want = set(expected)
    missing = sorted(want - have)
    extra = sorted(have - want)
    ignored = [n for n in extra if any(fnmatch.fnmatchcase(n, pat) for pat in ignore)]
    unexpected = [n for n in extra if n not in set(ignored)]
    wrong_shape, bad_dtype = [], []
    for name in sorted(want & have):
        if tuple(files.shape(name)) != tuple(expected[name].shape):
            wrong_shape.append((name, expected[name].shape, files.shape(name)))
        if not files.supported(name):
            bad_dtype.append((name, files.dtype_name(name)))
        elif expected[name].role != "table" and files.dtype_name(name) in ("I32", "I64"):
            bad_dtype.append((name, files.dtype_name(name)))
    if missing or unexpected or wrong_shape or bad_dtype:
        raise WeightError(files.model_dir, missing, unexpected, wrong_shape, bad_dtype)
    return ignored


def read_model_tensors(model_dir: str, expected: Mapping[str, TensorSpec], ignore=()) -> Iterator[tuple]:
    """Check the folder against `expected`, then yield (name, tensor) one at a time, each in
    the precision it was stored in (bfloat16 stays bfloat16, 32-bit stays 32-bit, integer
    tables int32).  Tensors that match `ignore` are left unread, with a warning."""
    files = ModelFiles(model_dir)
    try:
        ignored = check_tensors(files, expected, ignore)
        if ignored:
            warnings.warn(f"{model_dir}: tensors the model does not use were left unread: " + ", ".join(ignored),
                          stacklevel=2)
        for name in expected:
            yield name, files.tensor(name)
    finally:
        files.close()


# ----------------------------------------------------------------------------
# random weights
# ----------------------------------------------------------------------------

def _tensor_seed(seed: int, name: str) -> int:
    # keyed by name, so the numbers do not depend on the order tensors are made in
    return (int(seed) * 1_000_003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63 - 1)


def random_tensors(expected: Mapping[str, TensorSpec], seed: int, *, std: float = 0.02,
                   matrix_dtype: torch.dtype = torch.bfloat16, device="cpu",
                   norm_std: float = 0.0) -> Iterator[tuple]:
    """Yield (name, tensor): matrices ~ N(0, std) in `matrix_dtype`, biases ~ N(0, std) and
    norm weights 1 + N(0, norm_std) in float32 (exactly 1.0 by default), integer tables zero.
    With norm_std > 0 every norm weight differs from every other, so a test model shows a
    norm weight that was swapped, dropped or skipped."""
    device = torch.device(device)
    if device.type == "cuda":
        yield from _random_tensors_on_device(expected, seed, std, matrix_dtype, device, norm_std)
        return
    for name, spec in expected.items():
        gen = torch.Generator(device=device)
        gen.manual_seed(_tensor_seed(seed, name))
        if spec.role == "table":
            t = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32, device=device)
            if norm_std > 0.0:
                t += torch.empty(spec.shape, dtype=torch.float32, device=device).normal_(0.0, norm_std, generator=gen)
        elif spec.init == "zeros":
            t = torch.zeros(spec.shape, dtype=torch.float32, device=device)
        elif spec.init == "normal":
            t = torch.empty(spec.shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=gen)
        else:
            raise ValueError(f"{name}: unknown init {spec.init!r}")
        if spec.role == "matrix":
            t = t.to(matrix_dtype)
        yield name, t


def _random_tensors_on_device(expected, seed, std, matrix_dtype, device, norm_std) -> Iterator[tuple]:
    """The same on a CUDA device, filled by the library's own kernel: element i of a tensor is a
    function of (seed, tensor name, i) alone (`sampling.rng.normal` restates it), written in the
    precision the tensor is kept in.  The numbers are not those of the host generator above; a model
    made here is handed to a plain implementation through `state_dict()`."""
    from ..kernels import ops
    for name, spec in expected.items():
        key = _tensor_seed(seed, name)
        if spec.role == "table":
            t = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif spec.init == "zeros":
            t = torch.zeros(spec.shape, dtype=torch.float32, device=device)
        elif spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32, device=device)
            if norm_std > 0.0:
                ops.fill_normal(t, key, mean=1.0, std=norm_std)
        elif spec.init == "normal":
            t = torch.empty(spec.shape, dtype=matrix_dtype if spec.role == "matrix" else torch.float32, device=device)
            ops.fill_normal(t, key, mean=0.0, std=std)
        else:
            raise ValueError(f"{name}: unknown init {spec.init!r}")
        yield name, t


def write_random_model(model_dir: str, config, seed: int, *, std: float = 0.02,
                       matrix_dtype: torch.dtype = torch.bfloat16, norm_std: float = 0.0) -> str:
    """Random-weights mode: make a model folder (config.json, model.safetensors) from a
    typed config and a seed.  Returns the folder."""
    from ..config.registry import get_architecture
    from ..engine.model import declared_tensors

    arch = get_architecture(config.architecture)
    spec = arch.build_spec(config)
    expected = declared_tensors(spec)
    os.makedirs(model_dir, exist_ok=True)
    tensors = dict(random_tensors(expected, seed, std=std, matrix_dtype=matrix_dtype, norm_std=norm_std))
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
    return model_dir
