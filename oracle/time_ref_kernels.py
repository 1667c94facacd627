"""Times the reference's own CUDA attention kernels and its output projection
(oracle/_ref/libref_attn.so, built by oracle/build_ref.sh for sm_100) on the GPU of this
machine, for the BASELINE configurations they can run: BF16, head_dim 128, one sequence (one
token for the projection), contiguous cache. TEST INFRASTRUCTURE: the
numbers are reference points for comparison tables; nothing of the product uses this file.

usage: python oracle/time_ref_kernels.py
"""
from __future__ import annotations

import ctypes as C
import json
from pathlib import Path

import torch

REF = Path(__file__).resolve().parent / "_ref" / "libref_attn.so"
PROJ_CASES = [  # name, output rows (hidden), input columns, weight copies cycled
    ("qwen3-32b-oproj-5120x8192", 5120, 8192, 6),
    ("qwen3-4b-oproj-2560x4096", 2560, 4096, 24),
]
CASES = [  # name, query heads, kv heads, cached length, layer caches cycled
    ("qwen3-4b-bf16-b1-ctx1024", 32, 8, 1024, 36),
    ("qwen3-4b-bf16-b1-ctx4096", 32, 8, 4096, 16),
    ("qwen3-4b-bf16-b1-ctx32768", 32, 8, 32768, 8),
]


def main() -> None:
    ref = C.CDLL(str(REF))
    ref.ref_mha_bf16.restype = C.c_int
    ref.ref_mha_bf16.argtypes = [C.c_void_p] * 4 + [C.c_int64, C.c_void_p] + [C.c_int32] * 8 + [C.c_void_p]
    dev = torch.device("cuda:0")
    for name, hq, hkv, length, layers in CASES:
        kv_dim = hkv * 128
        q = torch.randn(hq * 128, device=dev).to(torch.bfloat16)
        k = torch.randn(layers, length, kv_dim, device=dev).to(torch.bfloat16)
        v = torch.randn(layers, length, kv_dim, device=dev).to(torch.bfloat16)
        out = torch.zeros(hq * 128, dtype=torch.bfloat16, device=dev)
        ws_floats = hq * ((length + 31) // 32) * 130
        ws = torch.zeros(ws_floats, dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream().cuda_stream

        def call(layer: int) -> None:
            rc = ref.ref_mha_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), ws.data_ptr(), ws_floats,
                                  out.data_ptr(), layers, layer, length - 1, kv_dim, hq // hkv, hq,
                                  128, length, stream)
            assert rc == 0, rc

        for i in range(5):
            call(i % layers)
        torch.cuda.synchronize()
        steps = 4 * layers
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            call(i % layers)
        stop.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(stop) * 1e3 / steps
        bytes_ = 2 * length * kv_dim * 2 + 2 * hq * 128 * 2
        print(json.dumps({"workload": name, "reference_cuda_us_per_layer": round(us, 2),
                          "algorithmic_gbs": round(bytes_ / us / 1e3, 1)}))


def projections() -> None:
    """kernel::fused_gemv_add_kernel_cu, one token, weights cycled over more copies than L2."""
    ref = C.CDLL(str(REF))
    ref.ref_fused_gemv_add.restype = C.c_int
    ref.ref_fused_gemv_add.argtypes = [C.c_void_p] * 3 + [C.c_int32] * 2 + [C.c_void_p]
    dev = torch.device("cuda:0")
    for name, n, k, copies in PROJ_CASES:
        x = torch.randn(k, device=dev).to(torch.bfloat16)
        ws = [(torch.randn(n, k, device=dev) / 64).to(torch.bfloat16) for _ in range(copies)]
        r = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        for w in ws:
            assert ref.ref_fused_gemv_add(x.data_ptr(), w.data_ptr(), r.data_ptr(), n, k, stream) == 0
        torch.cuda.synchronize()
        steps = 10 * copies
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            ref.ref_fused_gemv_add(x.data_ptr(), ws[i % copies].data_ptr(), r.data_ptr(), n, k, stream)
        stop.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(stop) * 1e3 / steps
        print(json.dumps({"workload": name, "reference_cuda_us": round(us, 2),
                          "algorithmic_gbs": round(n * k * 2 / us / 1e3, 1)}))


if __name__ == "__main__":
    projections()
    main()
