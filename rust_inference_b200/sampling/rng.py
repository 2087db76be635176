"""The sampler's counter-based uniform numbers, restated on the host.

The kernel draws u = f(seed, stream, counter) with `stream` the index of the sequence
among the requests and `counter` the number of tokens it has drawn so far; this is the
same function in Python, for tests and for anyone who wants to replay a draw.  The
reference steps one xorshift64 state through all draws (sampler.rs:213-218), which ties
a sequence's numbers to everything sampled before it.
"""
from __future__ import annotations

_M = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def uniform(seed: int, stream: int, counter: int) -> float:
    """u in (0, 1], a multiple of 2^-24."""
    z = _mix64((seed & _M) ^ _mix64(((stream & 0xFFFFFFFF) << 32) | (counter & 0xFFFFFFFF)))
    return ((z >> 40) + 1) / 16777216.0


def normal(key: int, index: int) -> float:
    """The standard normal number `ops.fill_normal` gives element `index` of a tensor keyed `key`
    (Box-Muller on two 24-bit uniforms of one 64-bit hash), in double precision."""
    import math
    z = _mix64((key & _M) ^ _mix64(index & _M))
    u1 = ((z >> 40) + 1) / 16777216.0
    u2 = ((z >> 16) & 0xFFFFFF) / 16777216.0
    return math.sqrt(-2.0 * math.log(u1)) * math.cos(2.0 * math.pi * u2)
