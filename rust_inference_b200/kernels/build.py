"""Compiling the native sources and loading them.

Each file under `csrc/` becomes one shared library with a plain C ABI, compiled the first
time something needs it and kept beside the sources (`csrc/_build/`), so a model only
compiles the kernels it runs: the CUDA sources by nvcc for sm_100a, the host runtime
(`host_runtime.cpp`: cache books, step packing) by the C++ compiler.  There is no other
implementation behind these libraries: if one cannot be built or loaded, the caller gets
the error.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

MODULES = {
    "elementwise": "elementwise.cu",
    "gemm_simt": "gemm_simt.cu",
    "attention_generic": "attention_generic.cu",
    "sampling": "sampling.cu",
    "gemm_tcgen05": "gemm_tcgen05.cu",
    "attention_mma": "attention_mma.cu",
    "attention_tcgen05": "attention_tcgen05.cu",
    "wait_probe": "wait_probe.cu",
    "host_runtime": "host_runtime.cpp",
}

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


CXX_FLAGS = ["-std=c++17", "-O2", "-shared", "-fPIC", "-fvisibility=hidden"]

# RI_B200_CHECK_BOUNDS=1: the checked build of the kernels (indices that reach memory through a table are
# compared with their limits, recorded and skipped when outside: `csrc/common.cuh`).  It is compiled into
# and loaded from a folder of its own, beside the ordinary libraries.
CHECKED = os.environ.get("RI_B200_CHECK_BOUNDS", "") == "1"

# RI_B200_TIMELINE=1: the timeline build (thread 0 of every launch's first block records when the kernel
# came onto an SM and when its wait for the kernel before ended: `csrc/common.cuh`), likewise in a
# folder of its own.  For looking at a step's kernels as they overlap; slightly slower than the ordinary one.
TIMELINE = os.environ.get("RI_B200_TIMELINE", "") == "1"


def _nvcc_flags(checked: bool, timeline: bool) -> list:
    return NVCC_FLAGS + (["-DRI_CHECK_BOUNDS"] if checked else []) + (["-DRI_TIMELINE"] if timeline else [])


class KernelBuildError(RuntimeError):
    pass


_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found: the sm_100a kernels cannot be compiled (set NVCC or PATH)")


def _cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("no C++ compiler found: the host runtime cannot be compiled (set CXX or PATH)")


def _build_dir(checked: bool | None = None, timeline: bool | None = None) -> str:
    checked = CHECKED if checked is None else checked
    timeline = TIMELINE if timeline is None else timeline
    d = os.environ.get("RI_B200_BUILD_DIR") or os.path.join(CSRC, "_build")
    if checked:
        d = os.path.join(d, "checked")
    if timeline:
        d = os.path.join(d, "timeline")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}_{threading.get_ident()}")      # several threads may ask at once
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"ri_b200_build_{os.getuid()}" + ("_checked" if checked else "")
                         + ("_timeline" if timeline else ""))
        os.makedirs(d, exist_ok=True)
        return d


def _source_digest(src: str, checked: bool, timeline: bool) -> str:
    h = hashlib.sha256()
    h.update(" ".join(_nvcc_flags(checked, timeline) if src.endswith(".cu") else CXX_FLAGS).encode())
    headers = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))) if src.endswith(".cu") else []
    for name in [src] + headers:
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    return h.hexdigest()


def _say(msg: str) -> None:
    print(f"[rust_inference_b200] {msg}", file=sys.stderr, flush=True)


def library_path(module: str, checked: bool | None = None, timeline: bool | None = None) -> str:
    return os.path.join(_build_dir(checked, timeline), f"libri_{module}.so")


def build(module: str, *, force: bool = False, verbose: bool = True, checked: bool | None = None,
          timeline: bool | None = None) -> str:
    """Compile one module if its library is missing or older than its sources (`checked`, `timeline`:
    that build instead of the one this process loads)."""
    checked = CHECKED if checked is None else checked
    timeline = TIMELINE if timeline is None else timeline
    if module not in MODULES:
        raise KernelBuildError(f"unknown kernel module {module!r}")
    src = MODULES[module]
    src_path = os.path.join(CSRC, src)
    if not os.path.isfile(src_path):
        raise KernelBuildError(f"kernel source {src_path} is missing")
    out = library_path(module, checked, timeline)
    stamp = out + ".sha256"
    digest = _source_digest(src, checked, timeline)
    lock_path = os.path.join(os.path.dirname(out), f".{module}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and os.path.isfile(out) and os.path.isfile(stamp):
                with open(stamp) as f:
                    if f.read().strip() == digest:
                        return out
            tmp = out + f".{os.getpid()}.tmp"
            if src.endswith(".cu"):
                cmd = [_nvcc()] + _nvcc_flags(checked, timeline) + ["-I", CSRC, "-o", tmp, src_path]
            else:
                cmd = [_cxx()] + CXX_FLAGS + ["-o", tmp, src_path]
            if verbose:
                _say(f"compiling {src}" + (" for sm_100a" + (" (checked build)" if checked else "")
                                            + (" (timeline build)" if timeline else "") + " ..."
                                            if src.endswith(".cu") else " ..."))
            t0 = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            last = t0
            while True:
                try:
                    output, _ = proc.communicate(timeout=5)
                    break
                except subprocess.TimeoutExpired:
                    if verbose and time.time() - last >= 15:
                        last = time.time()
                        _say(f"  still compiling {src} ({int(last - t0)} s)")
            if proc.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise KernelBuildError(f"the compiler failed on {src}:\n{' '.join(cmd)}\n{output}")
            os.replace(tmp, out)
            with open(stamp, "w") as f:
                f.write(digest)
            if verbose:
                _say(f"  built {os.path.basename(out)} in {time.time() - t0:.1f} s")
            return out
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def load(module: str) -> ctypes.CDLL:
    """The module's library, built first if need be.  Raises if it cannot be had."""
    with _lock:
        lib = _loaded.get(module)
        if lib is None:
            path = build(module)
            try:
                lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            lib.ri_last_error.restype = ctypes.c_char_p
            _loaded[module] = lib
        return lib


def loaded_cuda_modules() -> list[str]:
    """Names of the CUDA libraries loaded so far."""
    return [m for m in _loaded if MODULES[m].endswith(".cu")]


def build_all(verbose: bool = True, checked: bool | None = None, timeline: bool | None = None,
              jobs: int | None = None) -> list[str]:
    """Every module of one build, several compilers at a time (`jobs`; default: the machine's cores, 8 at most)."""
    from concurrent.futures import ThreadPoolExecutor
    names = [m for m in MODULES if os.path.isfile(os.path.join(CSRC, MODULES[m]))]
    jobs = jobs or max(1, min(8, os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        return list(pool.map(lambda m: build(m, verbose=verbose, checked=checked, timeline=timeline), names))
