"""Times the reference's own CUDA attention kernels (oracle/_ref/libref_attn.so, built by
oracle/build_ref.sh for sm_100) on the GPU of this machine, for the BASELINE configurations
they can run: BF16, head_dim 128, one sequence, contiguous cache. TEST INFRASTRUCTURE: the
numbers go into the comparison table of BASELINE.md; nothing of the product uses this file.

usage: python oracle/time_ref_kernels.py
"""
from __future__ import annotations

import ctypes as C
import json
from pathlib import Path

import torch

REF = Path(__file__).resolve().parent / "_ref" / "libref_attn.so"
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


if __name__ == "__main__":
    main()
