"""Seeded synthetic GGUF blocks and activations with the value distributions of the benchmark configs.

No model file is needed: every tensor is generated from a (seed, name) pair with numpy's Philox
generator, so the same bytes can be rebuilt on any machine. The block layouts are the plain GGUF ones:
Q8_0 = fp16 d + 32 int8 (34 B / 32 values); Q4_K = fp16 d, fp16 dmin, 12 B of packed 6-bit scales and
mins, 128 B of nibbles (144 B / 256); Q6_K = 128 B low nibbles, 64 B high bit pairs, 16 int8 scales,
fp16 d (210 B / 256).
"""
from __future__ import annotations

import zlib

import numpy as np

Q8_0, Q4_K, Q6_K = 8, 12, 14
BLOCK_VALUES = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210}
TYPE_NAMES = {Q8_0: "q8_0", Q4_K: "q4_k", Q6_K: "q6_k"}


def rng_for(seed: int, name: str) -> np.random.Generator:
    """A counter-based generator keyed by (seed, tensor name)."""
    return np.random.Generator(np.random.Philox(key=[seed & (2**64 - 1), zlib.crc32(name.encode())]))


def row_bytes(ggml_type: int, columns: int) -> int:
    values = BLOCK_VALUES[ggml_type]
    if columns <= 0 or columns % values:
        raise ValueError(f"{columns} columns are not a whole number of {values}-value blocks")
    return columns // values * BLOCK_BYTES[ggml_type]


def _half_bits(rng: np.random.Generator, count: int, low: float, high: float) -> np.ndarray:
    return rng.uniform(low, high, count).astype(np.float32).astype(np.float16).view(np.uint16)


def q8_0_blocks(rng, blocks: int, d_range=(1e-4, 1e-2)) -> np.ndarray:
    """int8 codes uniform in [-127, 127]; fp16 scale uniform in ``d_range``."""
    data = np.empty((blocks, 34), np.uint8)
    data[:, 0:2] = _half_bits(rng, blocks, *d_range).view(np.uint8).reshape(blocks, 2)
    data[:, 2:] = rng.integers(-127, 128, (blocks, 32), dtype=np.int8).view(np.uint8)
    return data.reshape(-1)


def q4_k_blocks(rng, blocks: int, d_range=(1e-4, 1e-3)) -> np.ndarray:
    """fp16 d and dmin uniform in ``d_range``; uniform random bytes for the packed 6-bit scales/mins and
    the nibbles, which makes every 6-bit field uniform in 0..63 and every code uniform in 0..15."""
    data = rng.integers(0, 256, (blocks, 144), dtype=np.uint8)
    data[:, 0:2] = _half_bits(rng, blocks, *d_range).view(np.uint8).reshape(blocks, 2)
    data[:, 2:4] = _half_bits(rng, blocks, *d_range).view(np.uint8).reshape(blocks, 2)
    return data.reshape(-1)


def q6_k_blocks(rng, blocks: int, d_range=(1e-4, 1e-3)) -> np.ndarray:
    """Uniform 6-bit codes (random ql/qh bytes), int8 scales uniform in [-32, 31], fp16 d in ``d_range``."""
    data = rng.integers(0, 256, (blocks, 210), dtype=np.uint8)
    data[:, 192:208] = rng.integers(-32, 32, (blocks, 16), dtype=np.int8).view(np.uint8)
    data[:, 208:210] = _half_bits(rng, blocks, *d_range).view(np.uint8).reshape(blocks, 2)
    return data.reshape(-1)


def matrix(ggml_type: int, rows: int, columns: int, seed: int, name: str = "w") -> np.ndarray:
    """Row-major [rows][columns] matrix of GGUF blocks as a flat uint8 array."""
    blocks = rows * (columns // BLOCK_VALUES[ggml_type])
    row_bytes(ggml_type, columns)
    rng = rng_for(seed, f"{name}:{TYPE_NAMES[ggml_type]}:{rows}x{columns}")
    if ggml_type == Q8_0:
        return q8_0_blocks(rng, blocks)
    if ggml_type == Q4_K:
        return q4_k_blocks(rng, blocks)
    if ggml_type == Q6_K:
        return q6_k_blocks(rng, blocks)
    raise ValueError(f"unsupported GGML type {ggml_type}")


def activations(tokens: int, columns: int, seed: int, name: str = "x") -> np.ndarray:
    """FP32 N(0,1) activations, [tokens][columns]."""
    return rng_for(seed, f"{name}:{tokens}x{columns}").standard_normal((tokens, columns), dtype=np.float32)


# Matrix sets of the benchmark configs: (name, type, rows, columns, copies per model).
QWEN25_05B_Q8 = [
    ("attn_q", Q8_0, 896, 896, 24), ("attn_k", Q8_0, 128, 896, 24), ("attn_v", Q8_0, 128, 896, 24),
    ("attn_o", Q8_0, 896, 896, 24), ("ffn_gate", Q8_0, 4864, 896, 24), ("ffn_up", Q8_0, 4864, 896, 24),
    ("ffn_down", Q8_0, 896, 4864, 24), ("lm_head", Q8_0, 151936, 896, 1),
]
QWEN25_7B_Q4KM = [
    ("attn_q", Q4_K, 3584, 3584, 28), ("attn_k", Q4_K, 512, 3584, 28), ("attn_v", Q6_K, 512, 3584, 28),
    ("attn_o", Q4_K, 3584, 3584, 28), ("ffn_gate", Q4_K, 18944, 3584, 28), ("ffn_up", Q4_K, 18944, 3584, 28),
    ("ffn_down", Q6_K, 3584, 18944, 28), ("lm_head", Q4_K, 152064, 3584, 1),
]
SHARDED_SWEEP = [
    ("ffn_up_70b", Q4_K, 28672, 8192, 1), ("ffn_down_70b", Q4_K, 8192, 28672, 1), ("lm_head_7b", Q4_K, 152064, 3584, 1),
]


def set_bytes(matrix_set) -> int:
    """Source GGUF bytes of one full pass over a matrix set (the algorithmic bytes of the roofline)."""
    return sum(rows * row_bytes(t, cols) * copies for _, t, rows, cols, copies in matrix_set)
