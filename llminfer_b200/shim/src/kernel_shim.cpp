// The reference's kernel entry points for the attention path, implemented on the C ABI of
// libgqa_b200.so. Signatures, argument meaning and failure behaviour (abort on a broken
// precondition) follow code/source/op/kernel/cuda/mha_kernel.cu:440-529,
// code/source/op/kernel/cuda/rmsnorm_kernel.cu:257-290,
// code/source/op/kernel/cuda/rope_kernel.cu:23-46 and, for the projection behind attention,
// code/source/op/kernel/cuda/matmul_kernel.cu:172-208, and in front of it, :247-298. This file only uses members that the
// reference's tensor::Tensor also has, so it compiles against either set of headers.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "base/alloc.h"
#include "gqa_b200.h"
#include "op/kernel_interface.h"

namespace {

void require(bool ok, const char* what) {
    if (!ok) {
        std::fprintf(stderr, "llminfer_b200 shim: check failed: %s\n", what);
        std::abort();
    }
}

void require_ok(int status, const char* where) {
    if (status != GQA_OK) {
        std::fprintf(stderr, "llminfer_b200 shim: %s failed: %s\n", where,
                     gqa_status_string(status));
        std::abort();
    }
}

int32_t dtype_code(base::DataType t) {
    return t == base::DataType::DataTypeFp32 ? GQA_DTYPE_F32 : GQA_DTYPE_BF16;
}

bool on_cuda(const tensor::Tensor& t) { return t.device_type() == base::DeviceType::DeviceCUDA; }

}  // namespace

namespace kernel {

void mha_kernel_cu(const tensor::Tensor& query, const tensor::Tensor& key_cache,
                   const tensor::Tensor& value_cache, const tensor::Tensor& kv_split_output,
                   const tensor::Tensor& output, int32_t layer_id, int32_t pos, int32_t kv_dim,
                   int32_t kv_mul, int32_t head_num, int32_t head_dim, int32_t max_seq_len,
                   void* stream) {
    require(!query.is_empty() && !key_cache.is_empty() && !value_cache.is_empty() &&
                !kv_split_output.is_empty() && !output.is_empty(), "tensors are not empty");
    // The reference's CUDA kernels take BF16 only; FP32 tensors (the shape its op tests use)
    // are served by the FP32 kernel of this library.
    const base::DataType io = query.data_type();
    require(io == base::DataType::DataTypeBf16 || io == base::DataType::DataTypeFp32,
            "query is BF16 or FP32");
    require(key_cache.data_type() == io && value_cache.data_type() == io &&
                output.data_type() == io, "caches and output share the query's data type");
    require(kv_split_output.data_type() == base::DataType::DataTypeFp32,
            "kv_split_output is FP32");
    require(on_cuda(query) && on_cuda(key_cache) && on_cuda(value_cache) &&
                on_cuda(kv_split_output) && on_cuda(output), "tensors live on the CUDA device");
    require(pos >= 0 && pos < max_seq_len, "0 <= pos < max_seq_len");
    require(head_dim == 128, "head_dim == 128");
    require(kv_mul > 0 && head_num % kv_mul == 0 && kv_dim == head_num / kv_mul * head_dim,
            "kv_dim == head_num / kv_mul * head_dim");
    const int32_t num_kv_heads = head_num / kv_mul;
    const int64_t layer_elems = static_cast<int64_t>(max_seq_len) * kv_dim;
    const int64_t layers = static_cast<int64_t>(key_cache.size()) / layer_elems;
    require(layers >= 1 && layer_id >= 0 && layer_id < layers, "layer_id inside the cache");

    gqa_decode_params p;
    std::memset(&p, 0, sizeof(p));
    p.dtype = dtype_code(io);
    p.batch = 1;
    p.num_q_heads = head_num;
    p.num_kv_heads = num_kv_heads;
    p.head_dim = head_dim;
    p.fixed_block = layer_id;
    require_ok(gqa_layout_reference(static_cast<int32_t>(layers), max_seq_len, num_kv_heads,
                                    head_dim, &p.layout), "gqa_layout_reference");
    p.q = query.ptr<void>();
    p.k_cache = key_cache.ptr<void>();
    p.v_cache = value_cache.ptr<void>();
    p.out = const_cast<void*>(output.ptr<void>());
    p.workspace = const_cast<void*>(kv_split_output.ptr<void>());
    p.workspace_bytes = kv_split_output.byte_size();
    const int32_t seq_len = pos + 1;
    p.seq_lens_host = &seq_len;
    p.stream = stream;
    // In the reference's decode step the kernels ahead of attention (QKV GEMV, QK-Norm + RoPE)
    // write the cache row of `pos` only (code/source/model/qwen3_fused.cpp:517-533), so older
    // rows may be fetched while they finish.
    p.early_prefetch = 1;
    require_ok(gqa_decode(&p), "gqa_decode");
}

void fused_qk_norm_rope_kernel_cu(const tensor::Tensor& query, const tensor::Tensor& key,
                                  const tensor::Tensor& weight, const tensor::Tensor& token_pos,
                                  const tensor::Tensor& sin_cache, const tensor::Tensor& cos_cache,
                                  int32_t dim, int32_t kv_dim, int32_t head_dim, void* stream) {
    require(query.data_type() == base::DataType::DataTypeBf16 &&
                key.data_type() == base::DataType::DataTypeBf16 &&
                weight.data_type() == base::DataType::DataTypeBf16, "query, key, weight are BF16");
    require(token_pos.data_type() == base::DataType::DataTypeInt32, "token_pos is INT32");
    require(sin_cache.data_type() == base::DataType::DataTypeFp32 &&
                cos_cache.data_type() == base::DataType::DataTypeFp32, "sin / cos are FP32");
    require(on_cuda(query) && on_cuda(key) && on_cuda(weight) && on_cuda(sin_cache) &&
                on_cuda(cos_cache), "tensors live on the CUDA device");
    require(token_pos.device_type() == base::DeviceType::DeviceCPU, "token_pos lives on the CPU");
    require(head_dim == 128, "head_dim == 128");
    const int32_t pos = token_pos.index<int32_t>(0);

    gqa_front_params f;
    std::memset(&f, 0, sizeof(f));
    f.batch = 1;
    f.num_q_heads = dim / head_dim;
    f.num_kv_heads = kv_dim / head_dim;
    f.head_dim = head_dim;
    f.table_len = static_cast<int32_t>(sin_cache.size() / (head_dim / 2));
    f.eps = 1e-6f;
    // `key` already is the cache row of this position (the QKV GEMV wrote it there): the key
    // is normalised and rotated in place and the value row is left alone.
    require_ok(gqa_layout_reference(1, 1, f.num_kv_heads, head_dim, &f.layout),
               "gqa_layout_reference");
    f.q = query.ptr<void>();
    f.q_out = const_cast<void*>(query.ptr<void>());
    f.k_new = key.ptr<void>();
    f.k_cache = const_cast<void*>(key.ptr<void>());
    f.qk_weight = weight.ptr<void>();
    f.sin_cache = sin_cache.ptr<float>();
    f.cos_cache = cos_cache.ptr<float>();
    f.positions_host = &pos;
    f.stream = stream;
    require_ok(gqa_qk_norm_rope_append(&f), "gqa_qk_norm_rope_append");
}

void sin_cos_cache_precompute_cu(const tensor::Tensor& sin_cache, const tensor::Tensor& cos_cache,
                                 int32_t head_dim, int32_t max_seq_len, void* stream) {
    require(!sin_cache.is_empty() && !cos_cache.is_empty(), "tables are not empty");
    require(sin_cache.data_type() == base::DataType::DataTypeFp32 &&
                cos_cache.data_type() == base::DataType::DataTypeFp32, "tables are FP32");
    require(on_cuda(sin_cache) && on_cuda(cos_cache), "tables live on the CUDA device");
    require_ok(gqa_sin_cos_cache(const_cast<float*>(sin_cache.ptr<float>()),
                                 const_cast<float*>(cos_cache.ptr<float>()), head_dim,
                                 max_seq_len, stream), "gqa_sin_cos_cache");
}

namespace {

// Scratch of the projection (per-KV-head sums in flight), owned by the shim the way the
// reference's model owns its buffers; one host thread drives the kernels, as in the reference.
void* projection_workspace(int which, size_t bytes, void* stream) {
    static void* ptrs[2] = {nullptr, nullptr};
    static size_t capacities[2] = {0, 0};
    void*& ptr = ptrs[which];
    size_t& capacity = capacities[which];
    if (bytes > capacity) {
        auto alloc = base::CUDADeviceAllocatorFactory::get_instance();
        if (ptr != nullptr) alloc->release(ptr);
        ptr = alloc->allocate(bytes);
        require(ptr != nullptr, "projection workspace allocated");
        alloc->memset_zero(ptr, bytes, stream, true);
        capacity = bytes;
    }
    return ptr;
}

}  // namespace

void fused_gemv_add_kernel_cu(const tensor::Tensor& input, const tensor::Tensor& weight,
                              const tensor::Tensor& output, void* stream) {
    require(!input.is_empty() && input.dims_size() == 1, "input is a vector");
    require(!weight.is_empty() && weight.dims_size() == 2, "weight is a matrix");
    require(!output.is_empty() && output.dims_size() == 1, "output is a vector");
    require(input.data_type() == base::DataType::DataTypeBf16 &&
                weight.data_type() == base::DataType::DataTypeBf16 &&
                output.data_type() == base::DataType::DataTypeBf16, "tensors are BF16");
    require(on_cuda(input) && on_cuda(weight) && on_cuda(output),
            "tensors live on the CUDA device");
    const int32_t n = weight.get_dim(0);
    const int32_t k = weight.get_dim(1);
    require(input.get_dim(0) == k && output.get_dim(0) == n, "shapes agree with the weight");
    require(k % 128 == 0 && n % 16 == 0, "columns are whole heads of 128, rows a multiple of 16");
    // Any grouping of the column heads gives the same sum up to FP32 rounding; take groups of
    // up to 8 heads.
    const int32_t heads = k / 128;
    int32_t per_group = 8;
    while (heads % per_group != 0) --per_group;

    gqa_oproj_params p;
    std::memset(&p, 0, sizeof(p));
    p.batch = 1;
    p.hidden = n;
    p.num_q_heads = heads;
    p.num_kv_heads = heads / per_group;
    p.head_dim = 128;
    p.weight_ld = k;
    p.attn_out = input.ptr<void>();
    p.weight = weight.ptr<void>();
    p.residual = const_cast<void*>(output.ptr<void>());
    p.workspace_bytes = gqa_oproj_workspace_bytes(n, p.num_kv_heads);
    p.workspace =
        p.workspace_bytes != 0 ? projection_workspace(0, p.workspace_bytes, stream) : nullptr;
    p.stream = stream;
    require_ok(gqa_oproj_residual(&p), "gqa_oproj_residual");
}

void fused_qkv_gemv_kernel_cu(const tensor::Tensor& input, const tensor::Tensor& weight,
                              const tensor::Tensor& query, const tensor::Tensor& key,
                              const tensor::Tensor& value, void* stream) {
    require(!input.is_empty() && input.dims_size() == 1, "input is a vector");
    require(!weight.is_empty() && weight.dims_size() == 2, "weight is a matrix");
    require(!query.is_empty() && query.dims_size() == 1 && !key.is_empty() &&
                key.dims_size() == 1 && !value.is_empty() && value.dims_size() == 1,
            "query, key, value are vectors");
    require(input.data_type() == base::DataType::DataTypeBf16 &&
                weight.data_type() == base::DataType::DataTypeBf16 &&
                query.data_type() == base::DataType::DataTypeBf16 &&
                key.data_type() == base::DataType::DataTypeBf16 &&
                value.data_type() == base::DataType::DataTypeBf16, "tensors are BF16");
    require(on_cuda(input) && on_cuda(weight) && on_cuda(query) && on_cuda(key) && on_cuda(value),
            "tensors live on the CUDA device");
    const int32_t hidden = input.get_dim(0);
    const int32_t dim = query.get_dim(0);
    const int32_t kv_dim = key.get_dim(0);
    require(value.get_dim(0) == kv_dim && weight.get_dim(0) == dim + 2 * kv_dim &&
                weight.get_dim(1) == hidden, "shapes agree with the weight");
    require(hidden % 128 == 0 && dim % 128 == 0 && kv_dim % 128 == 0, "whole heads of 128");

    gqa_qkv_params p;
    std::memset(&p, 0, sizeof(p));
    p.batch = 1;
    p.hidden = hidden;
    p.num_q_heads = dim / 128;
    p.num_kv_heads = kv_dim / 128;
    p.head_dim = 128;
    p.weight_ld = hidden;
    p.x = input.ptr<void>();
    p.weight = weight.ptr<void>();
    p.q_out = const_cast<void*>(query.ptr<void>());
    p.k_out = const_cast<void*>(key.ptr<void>());
    p.v_out = const_cast<void*>(value.ptr<void>());
    p.workspace_bytes = gqa_qkv_workspace_bytes(hidden, p.num_q_heads, p.num_kv_heads);
    p.workspace =
        p.workspace_bytes != 0 ? projection_workspace(1, p.workspace_bytes, stream) : nullptr;
    p.stream = stream;
    require_ok(gqa_qkv_gemv(&p), "gqa_qkv_gemv");
}

namespace {
[[noreturn]] void no_cpu_path(const char* op) {
    std::fprintf(stderr, "llminfer_b200 shim: %s has no kernel for this device type "
                         "(only DeviceCUDA is served)\n", op);
    std::abort();
}
}  // namespace

MHAKernel get_mha_kernel(base::DeviceType device_type) {
    if (device_type != base::DeviceType::DeviceCUDA) no_cpu_path("mha");
    return mha_kernel_cu;
}

FusedQKNormRoPEKernel get_fused_qk_norm_rope_kernel(base::DeviceType device_type) {
    if (device_type != base::DeviceType::DeviceCUDA) no_cpu_path("fused_qk_norm_rope");
    return fused_qk_norm_rope_kernel_cu;
}

FusedGEMVAddKernel get_fused_gemv_add_kernel(base::DeviceType device_type) {
    if (device_type != base::DeviceType::DeviceCUDA) no_cpu_path("fused_gemv_add");
    return fused_gemv_add_kernel_cu;
}

FusedQKVGEMVKernel get_fused_qkv_gemv_kernel(base::DeviceType device_type) {
    if (device_type != base::DeviceType::DeviceCUDA) no_cpu_path("fused_qkv_gemv");
    return fused_qkv_gemv_kernel_cu;
}

SinCosCacheKernel get_sin_cos_cache_kernel(base::DeviceType device_type) {
    if (device_type != base::DeviceType::DeviceCUDA) no_cpu_path("sin_cos_cache");
    return sin_cos_cache_precompute_cu;
}

}  // namespace kernel
