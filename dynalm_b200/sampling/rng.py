"""xoshiro256** seeded through splitmix64, one generator per request
(dynalm/src/sampling/sampler.cpp:55-81)."""

from __future__ import annotations

import os

_M = (1 << 64) - 1


def _rotl(x: int, k: int) -> int:
    return ((x << k) | (x >> (64 - k))) & _M


class Xoshiro256:
    def __init__(self, seed: int = None):
        if seed is None:
            seed = int.from_bytes(os.urandom(8), "little")
        x = seed & _M
        self.s = [0, 0, 0, 0]
        for i in range(4):
            x = (x + 0x9E3779B97F4A7C15) & _M
            z = x
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
            self.s[i] = z ^ (z >> 31)

    def next(self) -> int:
        s = self.s
        result = (_rotl((s[1] * 5) & _M, 7) * 9) & _M
        t = (s[1] << 17) & _M
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = _rotl(s[3], 45)
        return result

    def uniform(self) -> float:
        """In [0, 1) with 53 random bits."""
        return (self.next() >> 11) * (2.0 ** -53)
