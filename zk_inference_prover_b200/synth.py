"""Seeded synthetic inputs (SplitMix64, the same stream in every language): the columns the benchmark proves and the tests compare on."""
import numpy as np

P = 2**31 - 1
MASK = (1 << 64) - 1


def splitmix64(seed, n):
    """n outputs of SplitMix64 started at `seed` (vectorised)."""
    idx = np.arange(1, n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + idx * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def m31_column(seed, n):
    """n uniform values in [0, p) (value = next_u64 mod p)."""
    return (splitmix64(seed, n) % np.uint64(P)).astype(np.uint32)


def qm31_array(seed, n, nonzero=False):
    v = m31_column(seed, 4 * n).reshape(n, 4)
    if nonzero:
        z = ~v.any(axis=1)
        v[z, 0] = 1
    return v


def edge_m31_column(seed, n):
    """Random column salted with the edge values 0, 1, p-1."""
    v = m31_column(seed, n)
    k = splitmix64(seed ^ 0xABCDEF, n) % np.uint64(16)
    v[k == 0] = 0
    v[k == 1] = P - 1
    v[k == 2] = 1
    return v
