// Drives the operator shim the way the reference's model code and op tests do
// (code/source/model/qwen3_fused.cpp:517-553, test/test_op/test_op_mha.cpp:7-63): tensors are
// built with the CPU allocator, moved with to_cuda(), the QK-Norm-RoPE and attention layers
// run through forward(), and the attention output is written to a file for the test to
// compare with the CPU oracle.
//
// usage: shim_driver <dir> <head_num> <kv_head_num> <layer_num> <layer_id> <max_seq_len> <pos>
// <dir> holds raw BF16 files q.bin [dim], k.bin / v.bin [layer_num, max_seq_len, kv_dim]
// (the row of `pos` holding the raw, un-normalised key) and w.bin [256]; the driver writes
// out.bin [dim], q_rot.bin [dim] and k_row.bin [kv_dim].
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "op/kernel_interface.h"
#include "op/mha.h"
#include "op/qk_norm_rope.h"

namespace {

std::vector<uint16_t> read_file(const std::string& path, size_t count) {
    std::vector<uint16_t> data(count);
    FILE* f = std::fopen(path.c_str(), "rb");
    CHECK(f != nullptr);
    CHECK(std::fread(data.data(), sizeof(uint16_t), count, f) == count);
    std::fclose(f);
    return data;
}

void write_file(const std::string& path, const void* data, size_t bytes) {
    FILE* f = std::fopen(path.c_str(), "wb");
    CHECK(f != nullptr);
    CHECK(std::fwrite(data, 1, bytes, f) == bytes);
    std::fclose(f);
}

tensor::Tensor host_bf16(const std::vector<uint16_t>& data, std::vector<int32_t> dims) {
    auto alloc = base::CPUDeviceAllocatorFactory::get_instance();
    tensor::Tensor t(base::DataType::DataTypeBf16, std::move(dims), true, alloc);
    for (size_t i = 0; i < data.size(); ++i) t.index<uint16_t>(static_cast<int64_t>(i)) = data[i];
    return t;
}

}  // namespace

// "oproj dir n k": residual += x . W^T through kernel::get_fused_gemv_add_kernel, the way
// the reference's model calls its output projection.
int run_projection(const std::string& dir, int32_t n, int32_t k) {
    const auto cuda = base::DeviceType::DeviceCUDA;
    tensor::Tensor x = host_bf16(read_file(dir + "/x.bin", k), {k});
    tensor::Tensor w = host_bf16(read_file(dir + "/w.bin", static_cast<size_t>(n) * k), {n, k});
    tensor::Tensor r = host_bf16(read_file(dir + "/r.bin", n), {n});
    x.to_cuda();
    w.to_cuda();
    r.to_cuda();
    auto config = std::make_shared<kernel::CudaConfig>();
    config->create();
    for (int rep = 0; rep < 2; ++rep) {  // the second call reuses the shim's scratch
        if (rep == 1) {
            tensor::Tensor again = host_bf16(read_file(dir + "/r.bin", n), {n});
            again.to_cuda();
            r = again;
        }
        kernel::get_fused_gemv_add_kernel(cuda)(x, w, r, config->stream);
        CHECK(cudaStreamSynchronize(config->stream) == cudaSuccess);
    }
    r.to_cpu();
    write_file(dir + "/r_out.bin", r.ptr<uint16_t>(), r.byte_size());
    std::printf("shim_driver ok\n");
    return 0;
}

// "qkv dir hidden dim kv_dim": the packed QKV projection through
// kernel::get_fused_qkv_gemv_kernel.
int run_qkv(const std::string& dir, int32_t hidden, int32_t dim, int32_t kv_dim) {
    const auto cuda = base::DeviceType::DeviceCUDA;
    const int32_t rows = dim + 2 * kv_dim;
    tensor::Tensor x = host_bf16(read_file(dir + "/x.bin", hidden), {hidden});
    tensor::Tensor w =
        host_bf16(read_file(dir + "/w.bin", static_cast<size_t>(rows) * hidden), {rows, hidden});
    x.to_cuda();
    w.to_cuda();
    auto alloc = base::CUDADeviceAllocatorFactory::get_instance();
    tensor::Tensor q(base::DataType::DataTypeBf16, dim, true, alloc);
    tensor::Tensor k(base::DataType::DataTypeBf16, kv_dim, true, alloc);
    tensor::Tensor v(base::DataType::DataTypeBf16, kv_dim, true, alloc);
    auto config = std::make_shared<kernel::CudaConfig>();
    config->create();
    for (int rep = 0; rep < 2; ++rep) {
        kernel::get_fused_qkv_gemv_kernel(cuda)(x, w, q, k, v, config->stream);
        CHECK(cudaStreamSynchronize(config->stream) == cudaSuccess);
    }
    q.to_cpu();
    k.to_cpu();
    v.to_cpu();
    write_file(dir + "/q_out.bin", q.ptr<uint16_t>(), q.byte_size());
    write_file(dir + "/k_out.bin", k.ptr<uint16_t>(), k.byte_size());
    write_file(dir + "/v_out.bin", v.ptr<uint16_t>(), v.byte_size());
    std::printf("shim_driver ok\n");
    return 0;
}

int main(int argc, char** argv) {
    if (argc == 6 && std::string(argv[1]) == "qkv") {
        return run_qkv(argv[2], std::atoi(argv[3]), std::atoi(argv[4]), std::atoi(argv[5]));
    }
    if (argc == 5 && std::string(argv[1]) == "oproj") {
        return run_projection(argv[2], std::atoi(argv[3]), std::atoi(argv[4]));
    }
    if (argc != 8) {
        std::fprintf(stderr, "usage: %s dir head_num kv_head_num layer_num layer_id max_seq_len pos\n",
                     argv[0]);
        return 2;
    }
    const std::string dir = argv[1];
    const int32_t head_num = std::atoi(argv[2]), kv_heads = std::atoi(argv[3]);
    const int32_t layer_num = std::atoi(argv[4]), layer_id = std::atoi(argv[5]);
    const int32_t max_seq_len = std::atoi(argv[6]), pos = std::atoi(argv[7]);
    const int32_t head_dim = 128, dim = head_num * head_dim, kv_dim = kv_heads * head_dim;
    const int32_t kv_mul = head_num / kv_heads;
    const auto cuda = base::DeviceType::DeviceCUDA;
    const size_t cache_elems = static_cast<size_t>(layer_num) * max_seq_len * kv_dim;

    tensor::Tensor query = host_bf16(read_file(dir + "/q.bin", dim), {dim});
    tensor::Tensor key_cache =
        host_bf16(read_file(dir + "/k.bin", cache_elems), {layer_num, max_seq_len, kv_dim});
    tensor::Tensor value_cache =
        host_bf16(read_file(dir + "/v.bin", cache_elems), {layer_num, max_seq_len, kv_dim});
    tensor::Tensor weight = host_bf16(read_file(dir + "/w.bin", 2 * head_dim), {2 * head_dim});
    query.to_cuda();
    key_cache.to_cuda();
    value_cache.to_cuda();
    weight.to_cuda();

    auto cuda_alloc = base::CUDADeviceAllocatorFactory::get_instance();
    tensor::Tensor sin_cache(base::DataType::DataTypeFp32, max_seq_len, head_dim / 2, true, cuda_alloc);
    tensor::Tensor cos_cache(base::DataType::DataTypeFp32, max_seq_len, head_dim / 2, true, cuda_alloc);
    tensor::Tensor kv_split(base::DataType::DataTypeFp32, head_num, 4 * max_seq_len, true, cuda_alloc);
    tensor::Tensor output(base::DataType::DataTypeBf16, dim, true, cuda_alloc);
    auto cpu_alloc = base::CPUDeviceAllocatorFactory::get_instance();
    tensor::Tensor token_pos(base::DataType::DataTypeInt32, 1, true, cpu_alloc);
    token_pos.index<int32_t>(0) = pos;

    auto config = std::make_shared<kernel::CudaConfig>();
    config->create();
    kernel::get_sin_cos_cache_kernel(cuda)(sin_cache, cos_cache, head_dim, max_seq_len,
                                           config->stream);

    // The key row of this position inside the cache, as Model::slice_kv_cache hands it out.
    const int64_t row_off = (static_cast<int64_t>(layer_id) * max_seq_len + pos) * kv_dim;
    tensor::Tensor key_row(base::DataType::DataTypeBf16, kv_dim, false, nullptr,
                           key_cache.ptr<uint16_t>(row_off));
    key_row.set_device_type(cuda);

    op::QKNormRoPELaryer qk_layer(cuda, dim, kv_dim, head_dim);
    qk_layer.set_cuda_config(config);
    STATUS_CHECK(qk_layer.set_weight(0, weight));
    STATUS_CHECK(qk_layer.forward(query, key_row, token_pos, sin_cache, cos_cache, tensor::Tensor()));

    op::MultiHeadAttention mha(cuda, kv_dim, kv_mul, head_num, head_dim, max_seq_len);
    mha.set_cuda_config(config);
    mha.set_pos(pos);
    mha.set_layer_id(layer_id);
    STATUS_CHECK(mha.forward(query, key_cache, value_cache, kv_split, output));
    CHECK(cudaStreamSynchronize(config->stream) == cudaSuccess);

    // A wrong dtype is refused by check(), not by an abort.
    tensor::Tensor bad(base::DataType::DataTypeFp32, dim, true, cuda_alloc);
    base::Status refused = mha.forward(bad, key_cache, value_cache, kv_split, output);
    CHECK(!refused && refused.get_err_code() == base::StatusCode::InvalidArgument);

    output.to_cpu();
    query.to_cpu();
    tensor::Tensor row_copy = key_row.clone();
    row_copy.to_cpu();
    write_file(dir + "/out.bin", output.ptr<uint16_t>(), output.byte_size());
    write_file(dir + "/q_rot.bin", query.ptr<uint16_t>(), query.byte_size());
    write_file(dir + "/k_row.bin", row_copy.ptr<uint16_t>(), row_copy.byte_size());
    std::printf("shim_driver ok\n");
    return 0;
}
