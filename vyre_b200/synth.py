"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

bf16 tensors are carried as uint16 bit patterns (numpy has no bf16). The same bytes feed the CUDA path and the
CPU checker, so parity never depends on a framework's RNG.
"""
from __future__ import annotations

import numpy as np


def f32_to_bf16_bits(a) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (finite inputs)."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = bits + (np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def int4_linear_inputs(m: int, n: int, k: int, group: int = 128, seed: int = 0):
    """Config 2/3: X bf16 [m,k] ~ N(0,1); W packed u4 [n,k/2] values U{0..15} (zero point 8, k=2j in the low
    nibble of byte j); bf16 scale [n,k/group] ~ U[1e-3, 2e-2]."""
    rng = np.random.default_rng(seed)
    x = f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    w = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)  # two uniform nibbles per byte
    s = f32_to_bf16_bits(rng.uniform(1e-3, 2e-2, size=(n, k // group)).astype(np.float32))
    return x, w, s


def int8_weight_only_inputs(m: int = 16, n: int = 1024, k: int = 1024, seed: int = 0):
    """Config 1: X f32 [m,k] ~ N(0,1); W int8 [n,k] U[-127,127]; per-channel f32 scale U[1e-3,1e-2]."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = rng.uniform(1e-3, 1e-2, size=n).astype(np.float32)
    return x, w, s


def int8_dynamic_inputs(m: int, n: int, k: int, seed: int = 0):
    """Config 5: X bf16 [m,k] ~ N(0,1); W int8 [n,k] U[-127,127]; per-channel f32 scale."""
    rng = np.random.default_rng(seed)
    x = f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    s = rng.uniform(1e-3, 1e-2, size=n).astype(np.float32)
    return x, w, s


def moe_ffn_inputs(tokens: int, hidden: int, inter: int, experts: int, group: int = 128, seed: int = 0):
    """Config 4: tokens bf16 ~ N(0,1); router bf16 [E,hidden] ~ N(0,0.02); per expert w1/w3 u4 [inter,hidden],
    w2 u4 [hidden,inter], bf16 group scales U[1e-3,2e-2]. Stacked as w13 [E,2,inter,hidden/2], w2 [E,hidden,inter/2]."""
    rng = np.random.default_rng(seed)
    x = f32_to_bf16_bits(rng.standard_normal((tokens, hidden), dtype=np.float32))
    wr = f32_to_bf16_bits((rng.standard_normal((experts, hidden), dtype=np.float32) * np.float32(0.02)))
    w13 = rng.integers(0, 256, size=(experts, 2, inter, hidden // 2), dtype=np.uint8)
    s13 = f32_to_bf16_bits(rng.uniform(1e-3, 2e-2, size=(experts, 2, inter, hidden // group)).astype(np.float32))
    w2 = rng.integers(0, 256, size=(experts, hidden, inter // 2), dtype=np.uint8)
    s2 = f32_to_bf16_bits(rng.uniform(1e-3, 2e-2, size=(experts, hidden, inter // group)).astype(np.float32))
    return x, wr, w13, s13, w2, s2
