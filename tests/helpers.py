"""Shared helpers of the GPU parity tests: seeded inputs, uploads, error measures."""
from __future__ import annotations

import numpy as np
import torch

import cases
from oracle import oracle

D = 128
NAN_BITS = 0x7FC0  # BF16 quiet NaN, used to poison cache rows that must never be read


def bf16_tensor(bits: np.ndarray, device="cuda:0") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device).view(torch.bfloat16)


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


def f32_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def rand_bits(rng: np.random.Generator, shape) -> np.ndarray:
    return cases.to_bf16_bits(rng.standard_normal(shape, dtype=np.float32))


def errors(got: np.ndarray, want: np.ndarray):
    """(max abs error, max abs error / max |want|)."""
    diff = float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))))
    scale = float(np.max(np.abs(want)))
    return diff, diff / max(scale, 1e-30)


def bf16_ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance in BF16 units of last place between two finite BF16 bit arrays."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, 0x8000 - (x & 0x7FFF), 0x8000 + x)
    return np.abs(key(a_bits) - key(b_bits))


def oracle_reference_layout(q_bits, k_bits, v_bits, *, layer_id, length, hkv, max_seq_len, accum=1):
    return oracle.mha_reference_layout(q_bits, k_bits.reshape(-1), v_bits.reshape(-1),
                                       layer_id=layer_id, pos=length - 1, hkv=hkv,
                                       max_seq_len=max_seq_len, accum=accum)


def bf16_mismatches(got_bits: np.ndarray, want_bits: np.ndarray, ulp: int = 1,
                    abs_tol: float = 2e-5) -> np.ndarray:
    """Mask of values that are neither within `ulp` BF16 units in the last place nor within
    `abs_tol` in value (near zero a unit in the last place is smaller than the FP32 rounding
    of a long sum)."""
    import cases
    dist = bf16_ulp_distance(got_bits, want_bits)
    diff = np.abs(cases.bf16_bits_to_f32(got_bits) - cases.bf16_bits_to_f32(want_bits))
    return (dist > ulp) & (diff > abs_tol)
