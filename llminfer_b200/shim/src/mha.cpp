// op::MultiHeadAttention: same slots, checks and call as the reference
// (code/source/op/mha.cpp:5-66), dispatching to the B200 kernels through the kernel registry.
#include "op/mha.h"

#include "op/kernel_interface.h"

namespace op {

MultiHeadAttention::MultiHeadAttention(base::DeviceType device_type, int32_t kv_dim,
                                       int32_t kv_mul, int32_t head_num, int32_t head_dim,
                                       int32_t max_seq_len)
    : Layer(device_type, LayerType::LayerMHA, "MHA"), kv_dim_(kv_dim), kv_mul_(kv_mul),
      head_num_(head_num), head_dim_(head_dim), max_seq_len_(max_seq_len) {
    reset_inputs_size(4);
    reset_outputs_size(1);
}

base::Status MultiHeadAttention::check() const {
    struct Slot {
        const tensor::Tensor* tensor;
        const char* what;
    };
    base::Status status = check_tensor_with_dim(get_input(0), device_type_, data_type_,
                                                head_num_ * head_dim_);
    if (!status) {
        status.set_err_msg("query: " + status.get_err_msg());
        return status;
    }
    const Slot caches[] = {{&get_input(1), "key_cache: "}, {&get_input(2), "value_cache: "}};
    for (const Slot& s : caches) {
        status = check_tensor(*s.tensor, device_type_, data_type_);
        if (!status) {
            status.set_err_msg(s.what + status.get_err_msg());
            return status;
        }
    }
    // The caller allocates the KV-split scratch as FP32 [head_num, 4 * max_seq_len]
    // (code/source/model/qwen3_fused.cpp:502); the split plan is kept inside it.
    status = check_tensor_with_dim(get_input(3), device_type_, base::DataType::DataTypeFp32,
                                   head_num_, 4 * max_seq_len_);
    if (!status) {
        status.set_err_msg("kv_split_output: " + status.get_err_msg());
        return status;
    }
    status = check_tensor_with_dim(get_output(0), device_type_, data_type_, head_num_ * head_dim_);
    if (!status) status.set_err_msg("output: " + status.get_err_msg());
    return status;
}

base::Status MultiHeadAttention::forward() {
    base::Status status = check();
    if (!status) return status;
    if (device_type_ == base::DeviceType::DeviceCUDA) CHECK(cuda_config_ != nullptr);
    kernel::get_mha_kernel(device_type_)(get_input(0), get_input(1), get_input(2), get_input(3),
                                         get_output(0), layer_id_, pos_, kv_dim_, kv_mul_,
                                         head_num_, head_dim_, max_seq_len_,
                                         cuda_config_ ? cuda_config_->stream : nullptr);
    return base::error::success();
}

}  // namespace op
