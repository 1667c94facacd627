"""Seeded inputs of the golden cases, shared by the fixture generator and the tests.

Values follow the workload description of the decode-attention benchmark: q, K, V ~ N(0, 1)
from a fixed seed, rounded to BF16 (round to nearest even); QK-Norm weights are
1 + 0.05 * N(0, 1) as in the reference's own precision script
(test_kernel/test_qwen3_bf16_ops.py:861-862).
"""
from __future__ import annotations

import zlib

import numpy as np

SEED = 20260614
HEAD_DIM = 128

# name, query heads, kv heads, cached length (pos + 1), layers in the cache, layer read, max_seq_len
ATTN_CASES = [
    ("len1", 32, 8, 1, 1, 0, 64),
    ("len17", 32, 8, 17, 1, 0, 64),
    ("len128_single_pass", 32, 8, 128, 1, 0, 256),
    ("len129_first_split", 32, 8, 129, 1, 0, 256),
    ("len1024_qwen3_4b", 32, 8, 1024, 1, 0, 1024),
    ("len2048_layer2of3", 32, 8, 2048, 3, 2, 2048),
    ("len4000_tail", 32, 8, 4000, 1, 0, 4096),
    ("len512_group2", 16, 8, 512, 1, 0, 512),
    ("len777_group8", 64, 8, 777, 1, 0, 1024),
    ("len300_group5", 40, 8, 300, 2, 1, 512),
]

# name, query heads, kv heads, position
FRONT_CASES = [
    ("pos0", 32, 8, 0),
    ("pos5", 32, 8, 5),
    ("pos12345", 32, 8, 12345),
    ("pos4095_group8", 64, 8, 4095),
]
# Projections on either side of attention (single token, as the reference runs them).
# name, output rows (hidden), input columns (query heads * 128)
OPROJ_CASES = [
    ("qwen3_0.6b", 1024, 2048),
    ("qwen3_4b", 2560, 4096),
    ("small", 48, 256),
]
# name, hidden, query heads, kv heads
QKV_CASES = [
    ("qwen3_0.6b", 1024, 16, 8),
    ("qwen3_4b", 2560, 32, 8),
]
FRONT_TABLE_LEN = 16384
TABLE_ROWS = [0, 1, 2, 5, 100, 1023, 4095, 12345, 16383]


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """FP32 -> BF16 bit patterns, round to nearest even (inputs are finite)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (u >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(
        np.float32)


def _rng(kind: int, index: int) -> np.random.Generator:
    return np.random.default_rng([SEED, kind, index])


def attention_inputs(index: int):
    """Returns (q [hq, 128], k_cache, v_cache [layers, max_seq_len, kv_dim]) as BF16 bits.

    Only rows 0..pos of the layer that is read are filled; the rest of the cache is zero.
    """
    _, hq, hkv, length, layers, layer_id, max_seq_len = ATTN_CASES[index]
    rng = _rng(1, index)
    kv_dim = hkv * HEAD_DIM
    q = to_bf16_bits(rng.standard_normal((hq, HEAD_DIM), dtype=np.float32))
    k_cache = np.zeros((layers, max_seq_len, kv_dim), dtype=np.uint16)
    v_cache = np.zeros((layers, max_seq_len, kv_dim), dtype=np.uint16)
    k_cache[layer_id, :length] = to_bf16_bits(rng.standard_normal((length, kv_dim), dtype=np.float32))
    v_cache[layer_id, :length] = to_bf16_bits(rng.standard_normal((length, kv_dim), dtype=np.float32))
    return q, k_cache, v_cache


def front_inputs(index: int):
    """Returns (q [hq, 128], k [hkv, 128], weight [256]) as BF16 bits."""
    _, hq, hkv, _ = FRONT_CASES[index]
    rng = _rng(2, index)
    q = to_bf16_bits(rng.standard_normal((hq, HEAD_DIM), dtype=np.float32))
    k = to_bf16_bits(rng.standard_normal((hkv, HEAD_DIM), dtype=np.float32))
    w = to_bf16_bits(1.0 + 0.05 * rng.standard_normal(2 * HEAD_DIM, dtype=np.float32))
    return q, k, w


def oproj_inputs(index: int):
    """Returns (x [k], weight [n, k], residual [n]) as BF16 bits: x, residual ~ N(0, 1),
    weight ~ N(0, 1) / sqrt(k) so that the product is of unit scale."""
    _, n, k = OPROJ_CASES[index]
    rng = _rng(3, index)
    x = to_bf16_bits(rng.standard_normal(k, dtype=np.float32))
    w = to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) / np.float32(np.sqrt(k)))
    r = to_bf16_bits(rng.standard_normal(n, dtype=np.float32))
    return x, w, r


def qkv_inputs(index: int):
    """Returns (x [hidden], weight [(hq + 2 hkv) * 128, hidden]) as BF16 bits."""
    _, hidden, hq, hkv = QKV_CASES[index]
    rng = _rng(4, index)
    rows = (hq + 2 * hkv) * HEAD_DIM
    x = to_bf16_bits(rng.standard_normal(hidden, dtype=np.float32))
    w = to_bf16_bits(rng.standard_normal((rows, hidden), dtype=np.float32)
                     / np.float32(np.sqrt(hidden)))
    return x, w


def checksum(*arrays: np.ndarray) -> int:
    crc = 0
    for a in arrays:
        crc = zlib.crc32(np.ascontiguousarray(a).tobytes(), crc)
    return crc
