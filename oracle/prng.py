"""Input generators of the reference's own tests (TEST INFRASTRUCTURE ONLY).

SplitMix64 / SeedTree follow sources/TinyTitanValidation/Support/PRNG/
SplitMix64.swift:4-24 and SeedTree.swift:4-19; the LCG follows
tests/TinyTitan/CPUEngine/CPUBatchedPrefillTests.swift:171-175.
"""
from __future__ import annotations

import numpy as np

_M64 = (1 << 64) - 1


class SplitMix64:
    def __init__(self, seed: int):
        self.state = seed & _M64

    def next(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        return z ^ (z >> 31)

    def uniform(self, lo: float, hi: float) -> np.float32:
        u = np.float32(self.next() >> 40) / np.float32(1 << 24)
        return np.float32(lo) + (np.float32(hi) - np.float32(lo)) * u

    def uniform_array(self, n: int, lo: float, hi: float) -> np.ndarray:
        """n successive uniform() draws, vectorised: the state advances by a constant, so draw i is a
        function of state + (i + 1) * gamma (uint64 arithmetic wraps exactly like the scalar form)."""
        if n == 0:
            return np.zeros(0, np.float32)
        with np.errstate(over="ignore"):
            z = np.uint64(self.state) + (np.arange(1, n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15))
            self.state = int(z[-1])
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            z = z ^ (z >> np.uint64(31))
        u = (z >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24)
        return (np.float32(lo) + (np.float32(hi) - np.float32(lo)) * u).astype(np.float32)


def seed_tree_key(root: int, label: str) -> SplitMix64:
    h = 0xCBF29CE484222325
    for byte in label.encode("utf-8"):
        h ^= byte
        h = (h * 0x100000001B3) & _M64
    return SplitMix64(root ^ h)


class LCG:
    """seed = seed*1664525 + 1013904223 (mod 2^32); value = (int(seed>>20) % 2001 - 1000)/1000."""

    def __init__(self, seed: int):
        self.seed = seed & 0xFFFFFFFF

    def random(self) -> np.float32:
        self.seed = (self.seed * 1664525 + 1013904223) & 0xFFFFFFFF
        return np.float32((self.seed >> 20) % 2001 - 1000) / np.float32(1000)

    def array(self, n: int) -> np.ndarray:
        return np.array([self.random() for _ in range(n)], dtype=np.float32)
