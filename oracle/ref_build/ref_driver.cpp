// C entry points around the reference's own CUDA decode-attention path, so a test can feed
// it raw device pointers and read back "the reference's own attention output".
//
// TEST INFRASTRUCTURE ONLY. This file is compiled together with the reference's sources
// where they lie in the reference checkout (nothing is copied) into oracle/_ref/, by
// oracle/build_ref.sh. The product library never links or loads it.
//
// Wrapped reference functions (paths inside the reference project):
//   kernel::mha_kernel_cu                  code/source/op/kernel/cuda/mha_kernel.cu:440
//   kernel::fused_qk_norm_rope_kernel_cu   code/source/op/kernel/cuda/rmsnorm_kernel.cu:257
//   kernel::sin_cos_cache_precompute_cu    code/source/op/kernel/cuda/rope_kernel.cu:23
//   kernel::fused_gemv_add_kernel_cu       code/source/op/kernel/cuda/matmul_kernel.cu:172
//   kernel::fused_qkv_gemv_kernel_cu       code/source/op/kernel/cuda/matmul_kernel.cu:247
#include <cstdint>
#include <cuda_runtime.h>
#include <utility>
#include <vector>

#include "tensor/tensor.h"

namespace kernel {
void mha_kernel_cu(const tensor::Tensor& query, const tensor::Tensor& key_cache,
                   const tensor::Tensor& value_cache, const tensor::Tensor& kv_split_output,
                   const tensor::Tensor& output, int32_t layer_id, int32_t pos, int32_t kv_dim,
                   int32_t kv_mul, int32_t head_num, int32_t head_dim, int32_t max_seq_len,
                   void* stream);
void fused_qk_norm_rope_kernel_cu(const tensor::Tensor& query, const tensor::Tensor& key,
                                  const tensor::Tensor& weight, const tensor::Tensor& token_pos,
                                  const tensor::Tensor& sin_cache, const tensor::Tensor& cos_cache,
                                  int32_t dim, int32_t kv_dim, int32_t head_dim, void* stream);
void sin_cos_cache_precompute_cu(const tensor::Tensor& sin_cache, const tensor::Tensor& cos_cache,
                                 int32_t head_dim, int32_t max_seq_len, void* stream);
void fused_gemv_add_kernel_cu(const tensor::Tensor& input, const tensor::Tensor& weight,
                              const tensor::Tensor& output, void* stream);
void fused_qkv_gemv_kernel_cu(const tensor::Tensor& input, const tensor::Tensor& weight,
                              const tensor::Tensor& query, const tensor::Tensor& key,
                              const tensor::Tensor& value, void* stream);
}  // namespace kernel

namespace {

tensor::Tensor borrow(base::DataType dtype, std::vector<int32_t> dims, void* ptr,
                      base::DeviceType device) {
    tensor::Tensor t(dtype, std::move(dims), false, nullptr, ptr);
    t.set_device_type(device);
    return t;
}

}  // namespace

extern "C" {

// All pointers are device pointers. `workspace_floats` must be at least
// head_num * ceil((pos + 1) / 32) * (head_dim + 2): the reference writes one
// (O[head_dim], m, l) record per 32 keys per query head and does not check the size.
int ref_mha_bf16(void* query, void* key_cache, void* value_cache, void* workspace,
                 int64_t workspace_floats, void* output, int32_t layer_num, int32_t layer_id,
                 int32_t pos, int32_t kv_dim, int32_t kv_mul, int32_t head_num, int32_t head_dim,
                 int32_t max_seq_len, void* stream) {
    const int64_t splits = (static_cast<int64_t>(pos) + 1 + 31) / 32;
    if (workspace_floats < static_cast<int64_t>(head_num) * splits * (head_dim + 2)) {
        return -1;
    }
    // The reference computes layer offsets in int32.
    if (static_cast<int64_t>(layer_num) * max_seq_len * kv_dim >= (int64_t{1} << 31)) {
        return -2;
    }
    const auto cuda = base::DeviceType::DeviceCUDA;
    const auto bf16 = base::DataType::DataTypeBf16;
    tensor::Tensor q = borrow(bf16, {head_num * head_dim}, query, cuda);
    tensor::Tensor k = borrow(bf16, {layer_num, max_seq_len, kv_dim}, key_cache, cuda);
    tensor::Tensor v = borrow(bf16, {layer_num, max_seq_len, kv_dim}, value_cache, cuda);
    tensor::Tensor w = borrow(base::DataType::DataTypeFp32,
                              {head_num, static_cast<int32_t>(workspace_floats / head_num)},
                              workspace, cuda);
    tensor::Tensor o = borrow(bf16, {head_num * head_dim}, output, cuda);
    kernel::mha_kernel_cu(q, k, v, w, o, layer_id, pos, kv_dim, kv_mul, head_num, head_dim,
                          max_seq_len, stream);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// In place on `query` [dim] and `key` [kv_dim] (bf16), weight [2 * head_dim] bf16,
// sin/cos tables [max_seq_len, head_dim / 2] fp32, all on the device.
int ref_fused_qk_norm_rope(void* query, void* key, void* weight, int32_t pos, void* sin_cache,
                           void* cos_cache, int32_t dim, int32_t kv_dim, int32_t head_dim,
                           int32_t max_seq_len, void* stream) {
    const auto cuda = base::DeviceType::DeviceCUDA;
    const auto bf16 = base::DataType::DataTypeBf16;
    const auto fp32 = base::DataType::DataTypeFp32;
    int32_t pos_host = pos;
    tensor::Tensor q = borrow(bf16, {dim}, query, cuda);
    tensor::Tensor k = borrow(bf16, {kv_dim}, key, cuda);
    tensor::Tensor w = borrow(bf16, {2 * head_dim}, weight, cuda);
    tensor::Tensor p = borrow(base::DataType::DataTypeInt32, {1}, &pos_host,
                              base::DeviceType::DeviceCPU);
    tensor::Tensor s = borrow(fp32, {max_seq_len, head_dim / 2}, sin_cache, cuda);
    tensor::Tensor c = borrow(fp32, {max_seq_len, head_dim / 2}, cos_cache, cuda);
    kernel::fused_qk_norm_rope_kernel_cu(q, k, w, p, s, c, dim, kv_dim, head_dim, stream);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int ref_sin_cos_cache(void* sin_cache, void* cos_cache, int32_t head_dim, int32_t max_seq_len,
                      void* stream) {
    const auto cuda = base::DeviceType::DeviceCUDA;
    const auto fp32 = base::DataType::DataTypeFp32;
    tensor::Tensor s = borrow(fp32, {max_seq_len, head_dim / 2}, sin_cache, cuda);
    tensor::Tensor c = borrow(fp32, {max_seq_len, head_dim / 2}, cos_cache, cuda);
    kernel::sin_cos_cache_precompute_cu(s, c, head_dim, max_seq_len, stream);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// residual[n] = bf16(residual[n] + sum_k input[k] * weight[n, k]); all bf16 on the device.
int ref_fused_gemv_add(void* input, void* weight, void* residual, int32_t n, int32_t k,
                       void* stream) {
    const auto cuda = base::DeviceType::DeviceCUDA;
    const auto bf16 = base::DataType::DataTypeBf16;
    tensor::Tensor in = borrow(bf16, {k}, input, cuda);
    tensor::Tensor w = borrow(bf16, {n, k}, weight, cuda);
    tensor::Tensor out = borrow(bf16, {n}, residual, cuda);
    kernel::fused_gemv_add_kernel_cu(in, w, out, stream);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// weight [dim + 2 * kv_dim, hidden] -> query [dim], key [kv_dim], value [kv_dim]; all bf16.
int ref_fused_qkv_gemv(void* input, void* weight, void* query, void* key, void* value,
                       int32_t hidden, int32_t dim, int32_t kv_dim, void* stream) {
    const auto cuda = base::DeviceType::DeviceCUDA;
    const auto bf16 = base::DataType::DataTypeBf16;
    tensor::Tensor in = borrow(bf16, {hidden}, input, cuda);
    tensor::Tensor w = borrow(bf16, {dim + 2 * kv_dim, hidden}, weight, cuda);
    tensor::Tensor q = borrow(bf16, {dim}, query, cuda);
    tensor::Tensor k = borrow(bf16, {kv_dim}, key, cuda);
    tensor::Tensor v = borrow(bf16, {kv_dim}, value, cuda);
    kernel::fused_qkv_gemv_kernel_cu(in, w, q, k, v, stream);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"
