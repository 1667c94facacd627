#!/usr/bin/env bash
# Builds oracle/_ref/libref_attn.so: the reference's own CUDA decode-attention path
# (mha_kernel.cu, rmsnorm_kernel.cu, rope_kernel.cu, the projection GEMVs of
# matmul_kernel.cu that sit on either side of it, plus its tensor/buffer/allocator
# sources), compiled from the reference checkout where it lies, for sm_100, against the
# glog stand-in header in oracle/ref_build/. TEST INFRASTRUCTURE ONLY: it is the
# second parity checker ("the reference's own attention output"), never shipped or timed
# as the product.
#
# usage: oracle/build_ref.sh <path-to-reference-checkout>
set -euo pipefail
REF="${1:?path to the reference checkout}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
SRC="$REF/code/source"
"$NVCC" -std=c++17 -O3 --extra-device-vectorization -Xptxas=-O3 \
    -gencode arch=compute_100,code=sm_100 \
    -shared -Xcompiler -fPIC -w \
    -I"$HERE/ref_build" -I"$REF/code/include" -I"$SRC/op/kernel/cuda" \
    "$HERE/ref_build/ref_driver.cpp" \
    "$SRC/op/kernel/cuda/mha_kernel.cu" \
    "$SRC/op/kernel/cuda/rmsnorm_kernel.cu" \
    "$SRC/op/kernel/cuda/rope_kernel.cu" \
    "$SRC/op/kernel/cuda/matmul_kernel.cu" \
    "$SRC/tensor/tensor.cpp" \
    "$SRC/base/buffer.cpp" "$SRC/base/alloc.cpp" "$SRC/base/alloc_cpu.cpp" \
    "$SRC/base/alloc_cu.cpp" "$SRC/base/base.cpp" \
    -o "$OUT/libref_attn.so"
echo "built $OUT/libref_attn.so"
