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
        return np.array([self.uniform(lo, hi) for _ in range(n)], dtype=np.float32)


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
