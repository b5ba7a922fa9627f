"""Seeded synthetic inputs that reproduce bit-for-bit on any machine (integer hashing and exactly rounded
float operations only, no library transcendental), shared by the fixture generator and the tests."""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def mix64(z: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser on uint64 arrays."""
    z = z.astype(np.uint64)
    with np.errstate(over="ignore"):
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def hash_u01(seed: int, n: int, lane: int = 0) -> np.ndarray:
    """n doubles in [0, 1): top 53 bits of a counter hash keyed by (seed, lane)."""
    with np.errstate(over="ignore"):
        base = np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(lane) * np.uint64(0xD1B54A32D192ED03)
        z = mix64(base + (np.arange(n, dtype=np.uint64) + np.uint64(1)) * np.uint64(0xE7037ED1A0B428DB))
    return (z >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def normalish(seed: int, shape, sigma: float) -> np.ndarray:
    """float32 array, roughly N(0, sigma^2): an Irwin-Hall sum of 6 hashed uniforms, exactly reproducible."""
    n = int(np.prod(shape))
    s = np.zeros(n, dtype=np.float64)
    for lane in range(6):
        s += hash_u01(seed, n, lane)
    x = (s - 3.0) * (sigma * 1.4142135623730951)  # var of the sum is 6/12
    return x.astype(np.float32).reshape(shape)


def grid_logits(seed: int, shape, spread: float) -> np.ndarray:
    """float32 logits on a coarse grid (multiples of spread / 1000), so ties are common."""
    n = int(np.prod(shape))
    k = np.floor(hash_u01(seed, n, 7) * 2001.0) - 1000.0
    return (k.astype(np.float32) / np.float32(1000.0) * np.float32(spread)).reshape(shape)


def zipf_history(seed: int, rows: int, length: int, vocab: int, s: float = 1.1) -> np.ndarray:
    """[rows, length] int32 token ids with P(rank k) ~ k^-s over the vocabulary (rank k -> a hashed id)."""
    # inverse CDF of the continuous power law on [1, vocab + 1), floored: close to Zipf and exactly reproducible
    u = hash_u01(seed, rows * length, 11)
    a = 1.0 - s
    hi = float(vocab + 1) ** a
    rank = np.floor((1.0 + u * (hi - 1.0)) ** (1.0 / a)).astype(np.int64) - 1
    rank = np.clip(rank, 0, vocab - 1)
    # scatter ranks over the id space with a fixed odd multiplier (a bijection mod a power of two is not needed)
    ids = (rank * 2654435761 + seed) % vocab
    return ids.astype(np.int32).reshape(rows, length)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (round to nearest even), as uint16."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))
    return (r >> np.uint32(16)).astype(np.uint16)
