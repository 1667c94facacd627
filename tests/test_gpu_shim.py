"""The C++ operator shim driven the way the reference's model code drives its layers:
op::QKNormRoPELaryer::forward on (query, cache row) then op::MultiHeadAttention::forward on the
reference's cache layout, through kernel::get_*_kernel, checked against the CPU oracle."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

import cases
import helpers as H
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("head_num,kv_heads,layer_num,layer_id,max_seq_len,pos", [
    (32, 8, 2, 1, 1024, 777),     # Qwen3-4B shape, split path inside the reference's scratch
    (16, 8, 1, 0, 256, 100),      # short context, no split
    (64, 8, 1, 0, 4096, 4095),    # group 8, last position of the cache
])
def test_layers_forward(tmp_path, built_lib, head_num, kv_heads, layer_num, layer_id, max_seq_len, pos):
    from llminfer_b200 import build
    build.build_shim()
    driver = ROOT / "llminfer_b200" / "lib" / "shim_driver"
    assert driver.exists()
    rng = np.random.default_rng(pos)
    kv_dim = kv_heads * H.D
    q = H.rand_bits(rng, (head_num, H.D))
    k = H.rand_bits(rng, (layer_num, max_seq_len, kv_dim))
    v = H.rand_bits(rng, (layer_num, max_seq_len, kv_dim))
    k[layer_id, pos + 1:] = H.NAN_BITS
    v[layer_id, pos + 1:] = H.NAN_BITS
    w = cases.to_bf16_bits(1.0 + 0.05 * rng.standard_normal(256, dtype=np.float32))
    for name, arr in (("q", q), ("k", k), ("v", v), ("w", w)):
        arr.tofile(tmp_path / f"{name}.bin")
    run = subprocess.run([str(driver), str(tmp_path), str(head_num), str(kv_heads), str(layer_num),
                          str(layer_id), str(max_seq_len), str(pos)], capture_output=True,
                         text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    out = np.fromfile(tmp_path / "out.bin", dtype=np.uint16).reshape(head_num, H.D)
    q_rot = np.fromfile(tmp_path / "q_rot.bin", dtype=np.uint16).reshape(head_num, H.D)
    k_row = np.fromfile(tmp_path / "k_row.bin", dtype=np.uint16).reshape(kv_heads, H.D)

    sin, cos = oracle.sin_cos_cache(128, max_seq_len, form=1)
    want_q, want_k = oracle.qk_norm_rope(q, k[layer_id, pos].reshape(kv_heads, H.D), w, sin[pos],
                                         cos[pos], accum=1)
    assert H.bf16_ulp_distance(q_rot, want_q).max() <= 1
    assert H.bf16_ulp_distance(k_row, want_k).max() <= 1
    k[layer_id, pos] = k_row.reshape(-1)
    want = H.oracle_reference_layout(q_rot, k, v, layer_id=layer_id, length=pos + 1, hkv=kv_heads,
                                     max_seq_len=max_seq_len)
    abs_err, rel_err = H.errors(cases.bf16_bits_to_f32(out), want)
    assert abs_err <= 2e-2 and rel_err <= 1e-2, (abs_err, rel_err)


@pytest.mark.parametrize("n,k", [(1024, 2048), (2560, 4096), (48, 384)])
def test_fused_gemv_add_kernel(tmp_path, built_lib, n, k):
    """kernel::get_fused_gemv_add_kernel(DeviceCUDA) on the reference's tensors: the output
    projection with residual add, against the FP64 oracle."""
    from llminfer_b200 import build
    build.build_shim()
    driver = ROOT / "llminfer_b200" / "lib" / "shim_driver"
    rng = np.random.default_rng(n + k)
    x = cases.to_bf16_bits(rng.standard_normal(k, dtype=np.float32))
    w = cases.to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32) / np.float32(np.sqrt(k)))
    r = cases.to_bf16_bits(rng.standard_normal(n, dtype=np.float32))
    for name, arr in (("x", x), ("w", w), ("r", r)):
        arr.tofile(tmp_path / f"{name}.bin")
    run = subprocess.run([str(driver), "oproj", str(tmp_path), str(n), str(k)],
                         capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    got = np.fromfile(tmp_path / "r_out.bin", dtype=np.uint16)
    want = oracle.gemv_add(x, w, r, accum=1)
    assert not H.bf16_mismatches(got, want).any()
    assert (got != want).mean() <= 0.02


@pytest.mark.parametrize("hidden,hq,hkv", [(1024, 16, 8), (2560, 32, 8)])
def test_fused_qkv_gemv_kernel(tmp_path, built_lib, hidden, hq, hkv):
    """kernel::get_fused_qkv_gemv_kernel(DeviceCUDA) on the reference's tensors."""
    from llminfer_b200 import build
    build.build_shim()
    driver = ROOT / "llminfer_b200" / "lib" / "shim_driver"
    rng = np.random.default_rng(hidden + hq)
    dim, kv_dim = hq * 128, hkv * 128
    x = cases.to_bf16_bits(rng.standard_normal(hidden, dtype=np.float32))
    w = cases.to_bf16_bits(rng.standard_normal((dim + 2 * kv_dim, hidden), dtype=np.float32)
                           / np.float32(np.sqrt(hidden)))
    x.tofile(tmp_path / "x.bin")
    w.tofile(tmp_path / "w.bin")
    run = subprocess.run([str(driver), "qkv", str(tmp_path), str(hidden), str(dim), str(kv_dim)],
                         capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    want = oracle.qkv_gemv(x, w, dim, kv_dim, accum=1)
    for name, w64 in zip(("q", "k", "v"), want):
        got = np.fromfile(tmp_path / f"{name}_out.bin", dtype=np.uint16)
        assert not H.bf16_mismatches(got, w64.reshape(-1)).any(), name
        assert (got != w64.reshape(-1)).mean() <= 0.02, name
