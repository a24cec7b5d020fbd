"""Philox4x32-10 in numpy, and the dropout multiplier the training-mode kernels derive from
it: element (pair, c) of h uses word c % 4 of the block with counter (c // 4, pair, 0, 0) and
key (seed & 0xffffffff, seed >> 32); it is dropped iff that word < p * 2**32. Test-side
restatement of gemmallm_b200/csrc/philox.cuh (Salmon et al., SC'11)."""
import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, k0: int, k1: int):
    """c0, c1: uint64 arrays holding 32-bit counters. Returns four uint32 arrays."""
    c0 = c0.astype(np.uint64) & MASK
    c1 = c1.astype(np.uint64) & MASK
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    for _ in range(10):
        p0 = M0 * c0
        p1 = M1 * c2
        n0 = ((p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0)) & MASK
        n1 = p1 & MASK
        n2 = ((p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1)) & MASK
        n3 = p0 & MASK
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return [a.astype(np.uint32) for a in (c0, c1, c2, c3)]


def dropout_multiplier(pairs: int, f: int, p: float, seed: int) -> np.ndarray:
    """float32 [pairs, f]: 0 where dropped, 1/(1-p) where kept."""
    if p <= 0:
        return np.ones((pairs, f), dtype=np.float32)
    thresh = min(int(p * 4294967296.0), 4294967295)
    blocks = (f + 3) // 4
    c0 = np.tile(np.arange(blocks, dtype=np.uint64), pairs)
    c1 = np.repeat(np.arange(pairs, dtype=np.uint64), blocks)
    words = philox4x32_10(c0, c1, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    w = np.stack(words, axis=1).reshape(pairs, blocks * 4)[:, :f]
    scale = np.float32(1.0) / (np.float32(1.0) - np.float32(p))
    return np.where(w >= thresh, scale, np.float32(0.0)).astype(np.float32)
