"""xorshift64* generator of the reference (src/sample.c:9-23): state ``seed * 0x9e3779b97f4a7c15 +
0x1234567`` (a fixed constant if that is zero); a draw is ``(next >> 40) / 2^24`` in [0, 1)."""
import numpy as np

MASK = (1 << 64) - 1
MULT = 0x2545F4914F6CDD1D


def seed_state(seed: int) -> int:
    s = (int(seed) * 0x9E3779B97F4A7C15 + 0x1234567) & MASK
    return s if s else MULT


def next_state(s: int) -> int:
    s ^= s >> 12
    s ^= (s << 25) & MASK
    s ^= s >> 27
    return s


def uniform_of_state(s: int) -> np.float32:
    """The draw that follows from an already advanced state."""
    return np.float32(((s * MULT) & MASK) >> 40) / np.float32(16777216.0)


class Rng:
    def __init__(self, seed: int):
        self.state = seed_state(seed)

    def uniform(self) -> np.float32:
        self.state = next_state(self.state)
        return uniform_of_state(self.state)
