"""Oracle (test infrastructure): Philox4x32-10 counter-based generator (Salmon, Moraes, Dror, Shaw: "Parallel random
numbers: as easy as 1, 2, 3", SC'11), restated in numpy.  The reference draws its uniforms from torch's generator
(ultraviolet/model.py:1210, ultraviolet/perf.py:595), which is itself Philox4x32-10; the keying used here --
key = seed, counter = (step, row key) -- is this build's so that a sequence's stream is independent of its slot."""
import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = np.uint32(0x9E3779B9), np.uint32(0xBB67AE85)


def philox4x32_10(counter, key):
    c = [np.uint32(x) for x in counter]
    k0, k1 = np.uint32(key[0]), np.uint32(key[1])
    with np.errstate(over="ignore"):
        for _ in range(10):
            p0 = M0 * np.uint64(c[0])
            p1 = M1 * np.uint64(c[2])
            hi0, lo0 = np.uint32(p0 >> np.uint64(32)), np.uint32(p0 & np.uint64(0xFFFFFFFF))
            hi1, lo1 = np.uint32(p1 >> np.uint64(32)), np.uint32(p1 & np.uint64(0xFFFFFFFF))
            c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
            k0, k1 = np.uint32(k0 + W0), np.uint32(k1 + W1)
    return c


def uniform(seed: int, row_key: int, step: int) -> np.float32:
    """The sampler's uniform in [0, 1): top 24 bits of the first output word."""
    seed, row_key, step = int(seed) & (2**64 - 1), int(row_key) & (2**64 - 1), int(step) & (2**64 - 1)
    c = philox4x32_10([step & 0xFFFFFFFF, step >> 32, row_key & 0xFFFFFFFF, row_key >> 32],
                      [seed & 0xFFFFFFFF, seed >> 32])
    return np.float32(int(c[0]) >> 8) * np.float32(1.0 / 16777216.0)
