// op::QKNormRoPELaryer: same slots, checks and call as the reference
// (code/source/op/qk_norm_rope.cpp:5-70).
#include "op/qk_norm_rope.h"

#include "op/kernel_interface.h"

namespace op {

QKNormRoPELaryer::QKNormRoPELaryer(base::DeviceType device_type, int32_t dim, int32_t kv_dim,
                                   int32_t head_dim)
    : LayerParam(device_type, LayerType::LayerMatmul, false, "QK-Norm-RoPE"), dim_(dim),
      kv_dim_(kv_dim), head_dim_(head_dim) {
    reset_inputs_size(5);
    reset_weights_size(1);
    reset_outputs_size(1);  // unused; the base class forward() overloads bind one output
}

base::Status QKNormRoPELaryer::check() const {
    base::Status status = check_tensor_with_dim(get_input(0), device_type_, data_type_, dim_);
    if (!status) return status;
    status = check_tensor_with_dim(get_input(1), device_type_, data_type_, kv_dim_);
    if (!status) return status;
    // The position is read on the host (code/source/op/qk_norm_rope.cpp:30).
    status = check_tensor_with_dim(get_input(2), base::DeviceType::DeviceCPU,
                                   base::DataType::DataTypeInt32, 1);
    if (!status) return status;
    status = check_tensor(get_input(3), device_type_, base::DataType::DataTypeFp32);
    if (!status) return status;
    status = check_tensor(get_input(4), device_type_, base::DataType::DataTypeFp32);
    if (!status) return status;
    return check_tensor_with_dim(get_weight(0), device_type_, data_type_, 2 * head_dim_);
}

base::Status QKNormRoPELaryer::forward() {
    base::Status status = check();
    if (!status) return status;
    if (device_type_ == base::DeviceType::DeviceCUDA) CHECK(cuda_config_ != nullptr);
    kernel::get_fused_qk_norm_rope_kernel(device_type_)(
        get_input(0), get_input(1), get_weight(0), get_input(2), get_input(3), get_input(4), dim_,
        kv_dim_, head_dim_, cuda_config_ ? cuda_config_->stream : nullptr);
    return base::error::success();
}

}  // namespace op
