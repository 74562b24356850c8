"""Seeded synthetic inputs for the Q4 linear configurations (numpy only).

No public dataset is involved: the reference quotes no numbers on one for this path, and
the shapes come from its own model presets.  The generator is counter based so that any
language can reproduce it: a splitmix64 stream (same constants as the reference's sign
generator, crates/inference/src/quant/quarot/hadamard.rs:22,141-146) gives u64 values
``mix(seed + (i + 1) * gamma)``; two of them make one normal deviate by Box-Muller in f64,
cast to f32 at the end.
"""
from __future__ import annotations

import numpy as np

GAMMA = np.uint64(0x9E3779B97F4A7C15)
TAG_X, TAG_W, TAG_A, TAG_B, TAG_OUTLIER = 1, 2, 3, 4, 5


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def stream_u64(seed: int, n: int, start: int = 0) -> np.ndarray:
    """Elements [start, start + n) of the splitmix64 stream of `seed`."""
    with np.errstate(over="ignore"):
        idx = np.arange(start + 1, start + n + 1, dtype=np.uint64)
        return _mix(np.uint64(seed & (2 ** 64 - 1)) + idx * GAMMA)


def normal_f32(seed: int, n: int, std: float = 1.0, chunk: int = 1 << 22) -> np.ndarray:
    out = np.empty(n, np.float32)
    for s in range(0, n, chunk):
        c = min(chunk, n - s)
        u = stream_u64(seed, 2 * c, 2 * s)
        u1 = ((u[0::2] >> np.uint64(11)).astype(np.float64) + 1.0) * (1.0 / 9007199254740992.0)   # (0, 1]
        u2 = ((u[1::2] >> np.uint64(11)).astype(np.float64) + 1.0) * (1.0 / 9007199254740992.0)
        z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
        out[s:s + c] = (z * std).astype(np.float32)
    return out


def config_seed(config_index: int, tag: int, extra: int = 0) -> int:
    base = (config_index * int(GAMMA)) & (2 ** 64 - 1)
    return (base ^ tag ^ (extra << 8)) & (2 ** 64 - 1)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bf16, returned widened back to f32."""
    u = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> np.uint64(16)) & np.uint64(1)
    u = (u + np.uint64(0x7FFF) + lsb) & np.uint64(0xFFFF0000)
    return u.astype(np.uint32).view(np.float32)


def bf16_bits(x_rounded: np.ndarray) -> np.ndarray:
    return (x_rounded.astype(np.float32).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def activations(config_index: int, m: int, k: int, extra: int = 0) -> np.ndarray:
    return normal_f32(config_seed(config_index, TAG_X, extra), m * k, 1.0).reshape(m, k)


def weights(config_index: int, n: int, k: int, extra: int = 0) -> np.ndarray:
    return normal_f32(config_seed(config_index, TAG_W, extra), n * k, 0.02).reshape(n, k)


def lora_factors(config_index: int, rank: int, k: int, n: int, extra: int = 0):
    """A [rank, k] and B [n, rank], both ~N(0, 0.02^2), in the reference's storage layout."""
    a = normal_f32(config_seed(config_index, TAG_A, extra), rank * k, 0.02).reshape(rank, k)
    b = normal_f32(config_seed(config_index, TAG_B, extra), n * rank, 0.02).reshape(n, rank)
    return a, b


def outlier_channels(config_index: int, k: int, fraction: float = 0.01) -> np.ndarray:
    """floor(fraction * k) channel indices from a seeded Fisher-Yates shuffle."""
    cnt = int(fraction * k)
    r = stream_u64(config_seed(config_index, TAG_OUTLIER), k)
    perm = np.arange(k)
    for i in range(k - 1, 0, -1):
        j = int(r[i] % np.uint64(i + 1))
        perm[i], perm[j] = perm[j], perm[i]
    return np.sort(perm[:cnt])


# (k, n) of the large-layer decode set: q/o-like, kv-like, up-like and down-like projections
LARGE_LAYER_SHAPES = [(5120, 5120), (5120, 1024), (5120, 17408), (17408, 5120)]
QUAROT_DEFAULT_SEED = 0xCAFEBABEDEADBEEF   # converter default, crates/inference/src/quant/quarot/convert.rs:78-86


def algorithmic_bytes(m: int, n: int, k: int, rank: int = 0, x_bytes: int = 4) -> int:
    """Weights payload + LoRA factors + x + y, each counted once."""
    return n * (k // 32) * 20 + 4 * rank * (k + n) + m * k * x_bytes + m * n * 4


def algorithmic_flops(m: int, n: int, k: int, rank: int = 0) -> int:
    return 2 * m * n * k + 2 * m * rank * (k + n)
