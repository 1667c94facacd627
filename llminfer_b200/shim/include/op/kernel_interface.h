// Kernel registry entries of the attention path, with the reference's function-pointer types
// and getters (code/source/op/kernel/kernel_interface.h:132-139, :154-183,
// code/source/op/kernel/kernel_interface.cpp:160-190). The CUDA getters return the B200
// kernels of this library; there is no CPU path: asking for one aborts, which is what the
// reference does for a device it has no kernel for.
#ifndef LLMINFER_SHIM_OP_KERNEL_INTERFACE_H
#define LLMINFER_SHIM_OP_KERNEL_INTERFACE_H

#include "tensor/tensor.h"

namespace kernel {

// The live argument order is (query, key_cache, value_cache, kv_split_output, output, ...):
// that is what op::MultiHeadAttention passes (code/source/op/mha.cpp:54-56) and what
// mha_kernel_cu takes (code/source/op/kernel/cuda/mha_kernel.cuh:7-21).
using MHAKernel = void (*)(const tensor::Tensor& query, const tensor::Tensor& key_cache,
                           const tensor::Tensor& value_cache,
                           const tensor::Tensor& kv_split_output, const tensor::Tensor& output,
                           int32_t layer_id, int32_t pos, int32_t kv_dim, int32_t kv_mul,
                           int32_t head_num, int32_t head_dim, int32_t max_seq_len, void* stream);
MHAKernel get_mha_kernel(base::DeviceType device_type);

using FusedQKNormRoPEKernel = void (*)(const tensor::Tensor& query, const tensor::Tensor& key,
                                       const tensor::Tensor& weight,
                                       const tensor::Tensor& token_pos,
                                       const tensor::Tensor& sin_cache,
                                       const tensor::Tensor& cos_cache, int32_t dim,
                                       int32_t kv_dim, int32_t head_dim, void* stream);
FusedQKNormRoPEKernel get_fused_qk_norm_rope_kernel(base::DeviceType device_type);

using SinCosCacheKernel = void (*)(const tensor::Tensor& sin_cache, const tensor::Tensor& cos_cache,
                                   int32_t head_dim, int32_t max_seq_len, void* stream);
SinCosCacheKernel get_sin_cos_cache_kernel(base::DeviceType device_type);

// Output projection with residual add, the step behind attention
// (code/source/op/kernel/kernel_interface.h:53-59): output[n] += dot(input, weight[n]).
using FusedGEMVAddKernel = void (*)(const tensor::Tensor& input, const tensor::Tensor& weight,
                                    const tensor::Tensor& output, void* stream);
FusedGEMVAddKernel get_fused_gemv_add_kernel(base::DeviceType device_type);

// Packed QKV projection, the step in front of QK-Norm + RoPE
// (code/source/op/kernel/kernel_interface.h:72-80).
using FusedQKVGEMVKernel = void (*)(const tensor::Tensor& input, const tensor::Tensor& weight,
                                    const tensor::Tensor& query, const tensor::Tensor& key,
                                    const tensor::Tensor& value, void* stream);
FusedQKVGEMVKernel get_fused_qkv_gemv_kernel(base::DeviceType device_type);

// The functions behind the getters, exported with the reference's names so that the
// reference's own kernel_interface.cpp links against this library unchanged.
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

#endif  // LLMINFER_SHIM_OP_KERNEL_INTERFACE_H
