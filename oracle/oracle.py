"""Python face of the CPU oracle (``oracle/gqa_oracle.c``, ``oracle/proj_oracle.c``) and of the
reference-kernel build.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``. The product never imports it.

``build()`` compiles the C restatement with gcc into ``oracle/liboracle.so``.
``build_ref(reference_root)`` compiles the reference's own CUDA attention sources, where they
lie in the reference checkout, into ``oracle/_ref/libref_attn.so`` (see ``build_ref.sh``).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path
from typing import Optional, Sequence

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"
SRC = HERE / "gqa_oracle.c"
SOURCES = [SRC, HERE / "proj_oracle.c"]
REF_LIB = HERE / "_ref" / "libref_attn.so"

DTYPE_F32 = 0
DTYPE_BF16 = 1

_lib: Optional[C.CDLL] = None


def build(force: bool = False) -> Path:
    newest = max(src.stat().st_mtime for src in SOURCES)
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        # -ffp-contract=off: the restatements spell out every fused multiply-add themselves.
        subprocess.run(["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-Wall",
                        "-ffp-contract=off", *map(str, SOURCES), "-o", str(LIB), "-lm"],
                       check=True)
    return LIB


def build_ref(reference_root: str, force: bool = False) -> Optional[Path]:
    """Builds the reference's CUDA kernels for sm_100; returns None when the checkout is absent."""
    root = Path(reference_root)
    if not (root / "code" / "source" / "op" / "kernel" / "cuda" / "mha_kernel.cu").exists():
        return REF_LIB if REF_LIB.exists() else None
    if force or not REF_LIB.exists():
        subprocess.run(["bash", str(HERE / "build_ref.sh"), str(root)], check=True,
                       capture_output=True)
    return REF_LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        h = C.CDLL(str(LIB))
        h.oracle_gqa_decode.restype = C.c_int
        h.oracle_gqa_decode.argtypes = [
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
            C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_void_p,
            C.c_int32, C.c_int32, C.c_int]
        h.oracle_mha_kernel_cpu.restype = C.c_int
        h.oracle_mha_kernel_cpu.argtypes = [C.c_void_p] * 5 + [C.c_int32] * 7
        h.oracle_qk_norm_rope.restype = C.c_int
        h.oracle_qk_norm_rope.argtypes = [C.c_void_p] * 5 + [C.c_int, C.c_int, C.c_int,
                                                              C.c_float, C.c_int]
        h.oracle_sin_cos_cache.restype = C.c_int
        h.oracle_sin_cos_cache.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        h.oracle_f32_to_bf16.restype = None
        h.oracle_f32_to_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        h.oracle_bf16_to_f32.restype = None
        h.oracle_bf16_to_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        h.oracle_max_threads.restype = C.c_int
        h.oracle_set_threads.restype = None
        h.oracle_set_threads.argtypes = [C.c_int]
        h.oracle_gemv_add.restype = C.c_int
        h.oracle_gemv_add.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_int64, C.c_int]
        h.oracle_qkv_gemv.restype = C.c_int
        h.oracle_qkv_gemv.argtypes = [C.c_void_p] * 5 + [C.c_int] * 5
        _lib = h
    return _lib


def max_threads() -> int:
    return lib().oracle_max_threads()


def use_all_cores() -> int:
    """Lets the parallel loops use every core this process may run on, whatever
    OMP_NUM_THREADS says (torchrun exports 1). Returns the thread count."""
    import os
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_threads(cores)
    return max_threads()


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even FP32 -> BF16 bit patterns (uint16)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16(x.ctypes.data, out.ctypes.data, x.size)
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().oracle_bf16_to_f32(x.ctypes.data, out.ctypes.data, x.size)
    return out


def _dtype_of(a: np.ndarray) -> int:
    if a.dtype == np.float32:
        return DTYPE_F32
    if a.dtype == np.uint16:
        return DTYPE_BF16
    raise TypeError(f"oracle takes float32 or bf16-as-uint16 arrays, got {a.dtype}")


def gqa_decode(q: np.ndarray, k: np.ndarray, v: np.ndarray, seq_lens: Sequence[int], *, hkv: int,
               stride_block: int, stride_token: int, stride_head: int, block_tokens: int,
               block_table: Optional[np.ndarray] = None, fixed_block: int = 0, accum: int = 1,
               threads: int = 0) -> np.ndarray:
    """q [batch, hq, d]; k, v flat caches; returns FP32 [batch, hq, d]. accum 0 = FP32, 1 = FP64."""
    batch, hq, d = q.shape
    dt = _dtype_of(q)
    assert _dtype_of(k) == dt and _dtype_of(v) == dt
    q = np.ascontiguousarray(q)
    out = np.empty((batch, hq, d), dtype=np.float32)
    lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    bt_ptr, bps = None, 0
    if block_table is not None:
        block_table = np.ascontiguousarray(block_table, dtype=np.int32)
        bt_ptr, bps = block_table.ctypes.data, block_table.shape[1]
    rc = lib().oracle_gqa_decode(q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data, dt,
                                 accum, batch, hq, hkv, d, lens.ctypes.data, stride_block,
                                 stride_token, stride_head, block_tokens, bt_ptr, bps, fixed_block,
                                 threads)
    if rc != 0:
        raise ValueError("oracle_gqa_decode rejected its arguments")
    return out


def mha_reference_layout(q: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, *, layer_id: int,
                         pos: int, hkv: int, max_seq_len: int, accum: int = 1,
                         threads: int = 0) -> np.ndarray:
    """One sequence on the reference's [layer, max_seq_len, kv_dim] cache; q [hq, d]."""
    hq, d = q.shape
    kv_dim = hkv * d
    return gqa_decode(q[None], k_cache, v_cache, [pos + 1], hkv=hkv,
                      stride_block=max_seq_len * kv_dim, stride_token=kv_dim, stride_head=d,
                      block_tokens=max_seq_len, fixed_block=layer_id, accum=accum,
                      threads=threads)[0]


def mha_kernel_cpu(query: np.ndarray, key_cache: np.ndarray, value_cache: np.ndarray, *,
                   layer_id: int, pos: int, kv_dim: int, kv_mul: int, head_num: int,
                   head_dim: int, max_seq_len: int):
    """The reference CPU kernel's argument list; returns (output, score scratch)."""
    query = np.ascontiguousarray(query, dtype=np.float32)
    score = np.zeros((head_num, max_seq_len), dtype=np.float32)
    out = np.zeros(head_num * head_dim, dtype=np.float32)
    rc = lib().oracle_mha_kernel_cpu(query.ctypes.data, score.ctypes.data, key_cache.ctypes.data,
                                     value_cache.ctypes.data, out.ctypes.data, layer_id, pos,
                                     kv_dim, kv_mul, head_num, head_dim, max_seq_len)
    if rc != 0:
        raise ValueError("oracle_mha_kernel_cpu rejected its arguments")
    return out, score


def qk_norm_rope(query: np.ndarray, key: np.ndarray, weight: np.ndarray, sin_row: np.ndarray,
                 cos_row: np.ndarray, *, eps: float = 1e-6, accum: int = 0):
    """query [hq, d], key [hkv, d], weight [2 d] as bf16 bits; returns new (query, key)."""
    q = np.array(query, dtype=np.uint16, copy=True)
    k = np.array(key, dtype=np.uint16, copy=True)
    w = np.ascontiguousarray(weight, dtype=np.uint16)
    s = np.ascontiguousarray(sin_row, dtype=np.float32)
    c = np.ascontiguousarray(cos_row, dtype=np.float32)
    rc = lib().oracle_qk_norm_rope(q.ctypes.data, k.ctypes.data, w.ctypes.data, s.ctypes.data,
                                   c.ctypes.data, q.shape[0], k.shape[0], q.shape[1], eps, accum)
    if rc != 0:
        raise ValueError("oracle_qk_norm_rope rejected its arguments")
    return q, k


def sin_cos_cache(head_dim: int, max_seq_len: int, form: int = 1):
    s = np.empty((max_seq_len, head_dim // 2), dtype=np.float32)
    c = np.empty_like(s)
    rc = lib().oracle_sin_cos_cache(s.ctypes.data, c.ctypes.data, head_dim, max_seq_len, form)
    if rc != 0:
        raise ValueError("oracle_sin_cos_cache rejected its arguments")
    return s, c


def gemv_add(x_bits: np.ndarray, w_bits: np.ndarray, residual_bits: np.ndarray, *, accum: int = 1,
             k: Optional[int] = None):
    """Output projection with residual add. x [batch, k] or [k], weight [n, ld >= k],
    residual [batch, n] or [n], BF16 bits. accum 0: the reference kernel's FP32 order,
    1: FP64 dot products, both rounded to BF16 bits; 2: the FP64 sums, not rounded."""
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    r = np.array(residual_bits, dtype=np.uint16, copy=True)
    x2 = x.reshape(-1, x.shape[-1])
    batch, kk = x2.shape[0], (k if k is not None else x2.shape[1])
    n, ld = w.shape
    out64 = np.zeros((batch, n), dtype=np.float64)
    rc = lib().oracle_gemv_add(x2.ctypes.data, w.ctypes.data, r.ctypes.data, out64.ctypes.data,
                               batch, n, kk, ld, accum)
    if rc != 0:
        raise ValueError("oracle_gemv_add rejected its arguments")
    return out64.reshape(r.shape) if accum == 2 else r


def qkv_gemv(x_bits: np.ndarray, w_bits: np.ndarray, dim: int, kv_dim: int, *, accum: int = 1):
    """Packed QKV projection. x [batch, hidden] or [hidden]; weight [dim + 2 kv_dim, hidden].
    Returns (query, key, value) BF16 bits with x's leading shape."""
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    x2 = x.reshape(-1, x.shape[-1])
    batch, hidden = x2.shape
    assert w.shape == (dim + 2 * kv_dim, hidden)
    q = np.zeros((batch, dim), dtype=np.uint16)
    k = np.zeros((batch, kv_dim), dtype=np.uint16)
    v = np.zeros((batch, kv_dim), dtype=np.uint16)
    rc = lib().oracle_qkv_gemv(x2.ctypes.data, w.ctypes.data, q.ctypes.data, k.ctypes.data,
                               v.ctypes.data, batch, hidden, dim, kv_dim, accum)
    if rc != 0:
        raise ValueError("oracle_qkv_gemv rejected its arguments")
    lead = x.shape[:-1]
    return q.reshape(lead + (dim,)), k.reshape(lead + (kv_dim,)), v.reshape(lead + (kv_dim,))
