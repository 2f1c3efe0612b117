"""Helpers shared by the tests: the reference's seeded test values and small conversions."""
import numpy as np


def values(n: int, seed: int) -> np.ndarray:
    """Uniform values in [-1, 1) from a fixed seed: the generator of the reference's GPU tests
    (crates/tachyon/tests/common/mod.rs:68-78), xorshift64 with shifts 13, 7, 17, top 24 bits."""
    out = np.empty(n, np.float32)
    s = seed
    mask = (1 << 64) - 1
    for i in range(n):
        s ^= (s << 13) & mask
        s ^= s >> 7
        s ^= (s << 17) & mask
        out[i] = np.float32(s >> 40) / np.float32(1 << 23) - np.float32(1.0)
    return out


def values_fast(n: int, seed: int) -> np.ndarray:
    """A vectorised seeded stand-in for large inputs (numpy PCG64), uniform in [-1, 1)."""
    return np.random.default_rng(seed).uniform(-1.0, 1.0, n).astype(np.float32)


def f16(a: np.ndarray) -> np.ndarray:
    """f32 -> f16 bits (round to nearest even), as uint16."""
    return np.asarray(a, np.float32).astype(np.float16).view(np.uint16)


def f16_to_f32(bits: np.ndarray) -> np.ndarray:
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)


def q8_weights(rows: int, cols: int, seed: int):
    """The benchmark's weight distribution: int8 uniform in [-127, 127], f16 scales |N(0,1)|*0.02/127 per 32."""
    rng = np.random.default_rng(seed)
    w = rng.integers(-127, 128, size=(rows, cols), dtype=np.int8)
    s = f16(np.abs(rng.standard_normal((rows, cols // 32))).astype(np.float32) * np.float32(0.02 / 127))
    return w, s
