"""The generation loop's books: which request has generated what, who goes on, who fits the cache.

Kept by the native host runtime (`csrc/host_runtime.cpp`, `ri_gen_*`); this class is its face: it owns
the handle, passes arrays and turns error codes into exceptions.  The rules are the reference's
(model.rs:373-442: at most max_tokens tokens; a sampled stop id ends the sequence and is not emitted;
prompt and generated tokens form the history of the repetition window), kept per request of a batch,
plus "length" as the end of a sequence that has no position left in the cache.
"""
from __future__ import annotations

from ctypes import c_int, c_void_p

import numpy as np

LIVE, STOP, LENGTH = 0, 1, 2
REASONS = {STOP: "stop", LENGTH: "length"}

_lib = None


def _runtime():
    global _lib
    if _lib is None:
        from ..kernels import build
        lib = build.load("host_runtime")
        lib.ri_gen_create.restype = c_void_p
        lib.ri_gen_create.argtypes = [c_int, c_int, c_void_p, c_int, c_int]
        lib.ri_gen_destroy.restype = None
        lib.ri_gen_destroy.argtypes = [c_void_p]
        for name, args in (("add", [c_void_p, c_int]), ("admit", [c_void_p, c_int, c_int]),
                           ("goes_on", [c_int, c_void_p, c_void_p, c_void_p]),
                           ("book", [c_int, c_void_p, c_void_p, c_void_p]), ("token_count", [c_int]),
                           ("finish", [c_int]), ("tokens", [c_int, c_void_p, c_int]),
                           ("recent", [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p])):
            fn = getattr(lib, "ri_gen_" + name)
            fn.restype = c_int
            fn.argtypes = [c_void_p] + args
        _lib = lib
    return _lib


def _i32(values) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=np.int32).reshape(-1)


class GenerationBooks:
    def __init__(self, max_tokens: int, max_seq_len: int, stop_ids=(), keep_history: bool = False):
        self._rt = _runtime()
        stops = _i32(sorted(int(s) for s in stop_ids))
        self._h = c_void_p(self._rt.ri_gen_create(int(max_tokens), int(max_seq_len), stops.ctypes.data if stops.size else None,
                                                  stops.size, 1 if keep_history else 0))
        if not self._h:
            raise ValueError(self._rt.ri_last_error().decode())
        self.keep_history = keep_history

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                self._rt.ri_gen_destroy(h)
            except Exception:          # the interpreter is shutting down and the library is gone
                pass

    def _call(self, name: str, *args, error=ValueError) -> int:
        rc = getattr(self._rt, "ri_gen_" + name)(self._h, *args)
        if rc < 0:
            raise error(self._rt.ri_last_error().decode())
        return rc

    def add(self, prompt) -> int:
        """A new request; returns its index.  An empty prompt, or one longer than max_seq_len, is refused."""
        p = _i32(prompt)
        return self._call("add", p.ctypes.data if p.size else None, p.size)

    def admit(self, pager, first: int, max_batch: int | None) -> int:
        """How many requests, from `first` on, fit the cache together with all they may generate."""
        return self._call("admit", pager._h, int(first), int(max_batch or 0), error=RuntimeError)

    def goes_on(self, requests, drawn) -> list:
        """Per request: will it certainly be stepped again after its drawn-th token?"""
        idx, d = _i32(requests), _i32(drawn)
        flags = np.zeros(max(idx.size, 1), dtype=np.int32)
        self._call("goes_on", idx.size, idx.ctypes.data, d.ctypes.data, flags.ctypes.data)
        return flags[:idx.size].astype(bool).tolist()

    def book(self, requests, tokens) -> list:
        """Book one sampled token per request; per request LIVE (feed the token), STOP or LENGTH."""
        idx, t = _i32(requests), _i32(tokens)
        status = np.zeros(max(idx.size, 1), dtype=np.int32)
        self._call("book", idx.size, idx.ctypes.data, t.ctypes.data, status.ctypes.data)
        return status[:idx.size].tolist()

    def token_count(self, request: int) -> int:
        return self._call("token_count", int(request))

    def tokens(self, request: int) -> list:
        n = self.token_count(request)
        out = np.zeros(max(n, 1), dtype=np.int32)
        self._call("tokens", int(request), out.ctypes.data, n)
        return out[:n].tolist()

    def finish_reason(self, request: int) -> str | None:
        return REASONS.get(self._call("finish", int(request)))

    def recent(self, requests, keep: int) -> list:
        """The last `keep` ids of each request's history (prompt and generated tokens), as lists."""
        idx = _i32(requests)
        width = max(int(keep), 1)
        counts = np.zeros(max(idx.size, 1), dtype=np.int32)
        rows = np.zeros((max(idx.size, 1), width), dtype=np.int32)
        self._call("recent", idx.size, idx.ctypes.data, int(keep), width, counts.ctypes.data, rows.ctypes.data)
        return [rows[i, :counts[i]].tolist() for i in range(idx.size)]
