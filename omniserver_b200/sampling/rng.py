"""Counter-based uniforms for sampling: u = f(seed, request id, index of the generated token).

The reference samples with torch.multinomial from the global, unseeded generator
(omniserve/runners/multimodal.py:378-379), so its draws depend on what else ran.  A uniform that is
a pure function of (seed, request, step) makes a request's tokens independent of the batch it
was in and repeatable by a plain implementation.
"""

from __future__ import annotations

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def _fnv1a(s: str) -> int:
    h = 0xCBF29CE484222325
    for b in s.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return h


def uniform(seed: int, request_id: str, step: int) -> float:
    """A float in [0, 1) with 24 random bits (exact in float32)."""
    x = _splitmix64((seed & _MASK) ^ _fnv1a(request_id))
    x = _splitmix64(x ^ ((step * 0xD6E8FEB86659FD93) & _MASK))
    return (x >> 40) / float(1 << 24)
