// Operator base classes of the shim: slot handling, tensor checks and forward overloads.
#include "op/layer.h"

#include <cstdarg>

namespace op {

Layer::Layer(base::DeviceType device_type, LayerType layer_type, std::string layer_name)
    : device_type_(device_type), layer_type_(layer_type), layer_name_(std::move(layer_name)) {}

base::Status Layer::check() const {
    return base::error::function_not_implement("check() is not implemented for this layer");
}

base::Status Layer::forward() {
    return base::error::function_not_implement("forward() is not implemented for this layer");
}

base::Status Layer::check_tensor(const tensor::Tensor& tensor, base::DeviceType device_type,
                                 base::DataType data_type) const {
    if (tensor.is_empty()) return base::error::invalid_argument("The tensor parameter is empty.");
    if (tensor.device_type() != device_type) {
        return base::error::invalid_argument("The tensor has a wrong device type.");
    }
    if (tensor.data_type() != data_type) {
        return base::error::invalid_argument("The tensor has a wrong data type.");
    }
    return base::error::success();
}

base::Status Layer::check_tensor_with_dim(const tensor::Tensor& tensor,
                                          base::DeviceType device_type, base::DataType data_type,
                                          ...) const {
    base::Status status = check_tensor(tensor, device_type, data_type);
    if (!status) return status;
    std::va_list args;
    va_start(args, data_type);
    const int32_t rank = tensor.dims_size();
    for (int32_t i = 0; i < rank; ++i) {
        const int32_t want = va_arg(args, int32_t);
        if (want != tensor.get_dim(i)) {
            va_end(args);
            return base::error::invalid_argument("The tensor has a wrong dim in dim" +
                                                 std::to_string(i));
        }
    }
    va_end(args);
    return base::error::success();
}

void Layer::set_input(int32_t idx, const tensor::Tensor& input) {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < inputs_.size());
    inputs_[idx] = input;
}

void Layer::set_output(int32_t idx, const tensor::Tensor& output) {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < outputs_.size());
    outputs_[idx] = output;
}

tensor::Tensor& Layer::get_input(int32_t idx) {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < inputs_.size());
    return inputs_[idx];
}

tensor::Tensor& Layer::get_output(int32_t idx) {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < outputs_.size());
    return outputs_[idx];
}

const tensor::Tensor& Layer::get_input(int32_t idx) const {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < inputs_.size());
    return inputs_[idx];
}

const tensor::Tensor& Layer::get_output(int32_t idx) const {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < outputs_.size());
    return outputs_[idx];
}

base::Status Layer::bind_and_run(std::initializer_list<const tensor::Tensor*> inputs,
                                 const tensor::Tensor& output) {
    int32_t idx = 0;
    for (const tensor::Tensor* t : inputs) set_input(idx++, *t);
    set_output(0, output);
    return forward();
}

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& output1) {
    return bind_and_run({&input1}, output1);
}

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                            const tensor::Tensor& output1) {
    return bind_and_run({&input1, &input2}, output1);
}

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                            const tensor::Tensor& input3, const tensor::Tensor& output1) {
    return bind_and_run({&input1, &input2, &input3}, output1);
}

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                            const tensor::Tensor& input3, const tensor::Tensor& input4,
                            const tensor::Tensor& output1) {
    return bind_and_run({&input1, &input2, &input3, &input4}, output1);
}

base::Status Layer::forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                            const tensor::Tensor& input3, const tensor::Tensor& input4,
                            const tensor::Tensor& input5, const tensor::Tensor& output1) {
    return bind_and_run({&input1, &input2, &input3, &input4, &input5}, output1);
}

LayerParam::LayerParam(base::DeviceType device_type, LayerType layer_type, bool is_quant_layer,
                       std::string layer_name)
    : Layer(device_type, layer_type, std::move(layer_name)), is_quant_layer_(is_quant_layer) {}

tensor::Tensor& LayerParam::get_weight(int32_t idx) {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < weights_.size());
    return weights_[idx];
}

const tensor::Tensor& LayerParam::get_weight(int32_t idx) const {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < weights_.size());
    return weights_[idx];
}

base::Status LayerParam::set_weight(int32_t idx, const tensor::Tensor& weight) {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < weights_.size());
    if (weight.data_type() != data_type_) {
        return base::error::invalid_argument("The weight has a wrong data type.");
    }
    weights_[idx] = weight;
    return base::error::success();
}

base::Status LayerParam::set_weight(int32_t idx, const std::vector<int32_t>& dims,
                                    const void* weight_ptr, base::DeviceType device_type) {
    CHECK(idx >= 0 && static_cast<size_t>(idx) < weights_.size());
    CHECK(weight_ptr != nullptr);
    tensor::Tensor weight(data_type_, dims, false, nullptr, const_cast<void*>(weight_ptr));
    weight.set_device_type(device_type);
    weights_[idx] = weight;
    return base::error::success();
}

}  // namespace op
