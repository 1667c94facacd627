"""Generates tests/golden/ref_cuda_bf16.npz (attention, front stage, tables) and
tests/golden/ref_cuda_proj.npz (the projection GEMVs on either side of attention) from the
reference's own CUDA kernels.

Runs on a machine with a GPU and oracle/_ref/libref_attn.so (built beforehand by
oracle/build_ref.sh from the reference checkout; the checkout itself is not needed at run
time). For every case in cases.py it feeds the seeded inputs to the reference's
kernel::mha_kernel_cu / fused_qk_norm_rope_kernel_cu / sin_cos_cache_precompute_cu and stores
their outputs, together with a checksum of the inputs so that a drifting random generator is
noticed. The oracle and the CUDA kernels of this repository are then tested against the file.

usage: python tests/golden/make_golden.py [attn|proj|all]
"""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402

REF = HERE.parent.parent / "oracle" / "_ref" / "libref_attn.so"


def up(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16)).to("cuda:0").view(torch.bfloat16)


def down(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def projections(ref) -> None:
    """kernel::fused_gemv_add_kernel_cu and kernel::fused_qkv_gemv_kernel_cu outputs."""
    ref.ref_fused_gemv_add.restype = C.c_int
    ref.ref_fused_gemv_add.argtypes = [C.c_void_p] * 3 + [C.c_int32] * 2 + [C.c_void_p]
    ref.ref_fused_qkv_gemv.restype = C.c_int
    ref.ref_fused_qkv_gemv.argtypes = [C.c_void_p] * 5 + [C.c_int32] * 3 + [C.c_void_p]
    store = {}
    for i, (name, n, k) in enumerate(cases.OPROJ_CASES):
        x, w, r = cases.oproj_inputs(i)
        dx, dw, dr = up(x), up(w), up(r).clone()
        rc = ref.ref_fused_gemv_add(dx.data_ptr(), dw.data_ptr(), dr.data_ptr(), n, k, None)
        torch.cuda.synchronize()
        assert rc == 0, (name, rc)
        store[f"oproj/{name}/out"] = down(dr)
        store[f"oproj/{name}/crc"] = np.array([cases.checksum(x, w, r)], dtype=np.uint64)
    for i, (name, hidden, hq, hkv) in enumerate(cases.QKV_CASES):
        x, w = cases.qkv_inputs(i)
        dim, kv_dim = hq * cases.HEAD_DIM, hkv * cases.HEAD_DIM
        dx, dw = up(x), up(w)
        q = torch.zeros(dim, dtype=torch.bfloat16, device="cuda:0")
        k = torch.zeros(kv_dim, dtype=torch.bfloat16, device="cuda:0")
        v = torch.zeros(kv_dim, dtype=torch.bfloat16, device="cuda:0")
        rc = ref.ref_fused_qkv_gemv(dx.data_ptr(), dw.data_ptr(), q.data_ptr(), k.data_ptr(),
                                    v.data_ptr(), hidden, dim, kv_dim, None)
        torch.cuda.synchronize()
        assert rc == 0, (name, rc)
        store[f"qkv/{name}/q"], store[f"qkv/{name}/k"], store[f"qkv/{name}/v"] = down(q), down(k), down(v)
        store[f"qkv/{name}/crc"] = np.array([cases.checksum(x, w)], dtype=np.uint64)
    np.savez_compressed(HERE / "ref_cuda_proj.npz", **store)
    print("wrote", HERE / "ref_cuda_proj.npz", "with", len(store), "arrays")


def main() -> None:
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    ref = C.CDLL(str(REF))
    if what in ("proj", "all"):
        projections(ref)
    if what == "proj":
        return
    out_path = HERE / "ref_cuda_bf16.npz"
    ref.ref_mha_bf16.restype = C.c_int
    ref.ref_mha_bf16.argtypes = [C.c_void_p] * 4 + [C.c_int64, C.c_void_p] + [C.c_int32] * 8 + [C.c_void_p]
    ref.ref_fused_qk_norm_rope.restype = C.c_int
    ref.ref_fused_qk_norm_rope.argtypes = [C.c_void_p] * 3 + [C.c_int32] + [C.c_void_p] * 2 + [C.c_int32] * 4 + [C.c_void_p]
    ref.ref_sin_cos_cache.restype = C.c_int
    ref.ref_sin_cos_cache.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    dev = torch.device("cuda:0")
    store = {}

    for i, (name, hq, hkv, length, layers, layer_id, max_seq_len) in enumerate(cases.ATTN_CASES):
        q, k, v = cases.attention_inputs(i)
        dq, dk, dv = up(q), up(k), up(v)
        out = torch.zeros(hq * cases.HEAD_DIM, dtype=torch.bfloat16, device=dev)
        splits = (length + 31) // 32
        ws_floats = hq * max(splits * (cases.HEAD_DIM + 2), 4 * max_seq_len)
        ws = torch.zeros(ws_floats, dtype=torch.float32, device=dev)
        rc = ref.ref_mha_bf16(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws_floats,
                              out.data_ptr(), layers, layer_id, length - 1, hkv * cases.HEAD_DIM,
                              hq // hkv, hq, cases.HEAD_DIM, max_seq_len, None)
        torch.cuda.synchronize()
        assert rc == 0, (name, rc)
        store[f"attn/{name}/out"] = down(out).reshape(hq, cases.HEAD_DIM)
        store[f"attn/{name}/crc"] = np.array([cases.checksum(q, k, v)], dtype=np.uint64)

    sin = torch.zeros(cases.FRONT_TABLE_LEN, cases.HEAD_DIM // 2, dtype=torch.float32, device=dev)
    cos = torch.zeros_like(sin)
    rc = ref.ref_sin_cos_cache(sin.data_ptr(), cos.data_ptr(), cases.HEAD_DIM, cases.FRONT_TABLE_LEN, None)
    torch.cuda.synchronize()
    assert rc == 0
    rows = torch.tensor(cases.TABLE_ROWS, device=dev)
    store["table/sin_rows"] = sin[rows].cpu().numpy()
    store["table/cos_rows"] = cos[rows].cpu().numpy()
    store["table/sin_sum"] = np.array([sin.double().sum().item()])
    store["table/cos_sum"] = np.array([cos.double().sum().item()])

    for i, (name, hq, hkv, pos) in enumerate(cases.FRONT_CASES):
        q, k, w = cases.front_inputs(i)
        dq, dk, dw = up(q).reshape(-1).clone(), up(k).reshape(-1).clone(), up(w)
        rc = ref.ref_fused_qk_norm_rope(dq.data_ptr(), dk.data_ptr(), dw.data_ptr(), pos,
                                        sin.data_ptr(), cos.data_ptr(), hq * cases.HEAD_DIM,
                                        hkv * cases.HEAD_DIM, cases.HEAD_DIM, cases.FRONT_TABLE_LEN,
                                        None)
        torch.cuda.synchronize()
        assert rc == 0, (name, rc)
        store[f"front/{name}/q"] = down(dq).reshape(hq, cases.HEAD_DIM)
        store[f"front/{name}/k"] = down(dk).reshape(hkv, cases.HEAD_DIM)
        store[f"front/{name}/sin"] = sin[pos].cpu().numpy()
        store[f"front/{name}/cos"] = cos[pos].cpu().numpy()
        store[f"front/{name}/crc"] = np.array([cases.checksum(q, k, w)], dtype=np.uint64)

    out_path.parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(out_path, **store)
    print("wrote", out_path, "with", len(store), "arrays")


if __name__ == "__main__":
    main()
