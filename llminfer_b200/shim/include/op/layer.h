// Operator base classes of the reference (code/include/op/layer.h:22-156), reduced to the
// members the attention operators and their callers use: numbered input / output / weight
// slots, check helpers, the forward() overloads that bind slots and run, and the CUDA stream
// holder.
#ifndef LLMINFER_SHIM_OP_LAYER_H
#define LLMINFER_SHIM_OP_LAYER_H

#include <initializer_list>
#include <memory>
#include <string>
#include <vector>

#include "base/cuda_config.h"
#include "tensor/tensor.h"

namespace op {

enum class LayerType : uint8_t {
    LayerUnknown = 0,
    LayerLinear = 1,
    LayerEncode = 2,
    LayerEmbedding = 3,
    LayerRMSNorm = 4,
    LayerMatmul = 5,
    LayerRoPE = 6,
    LayerMHA = 7,
    LayerSoftmax = 8,
    LayerAdd = 9,
    LayerSwiGLU = 10,
};

class Layer {
public:
    explicit Layer(base::DeviceType device_type, LayerType layer_type, std::string layer_name = "");
    virtual ~Layer() = default;

    virtual base::Status init() { return base::error::success(); }
    virtual base::Status check() const;
    virtual base::Status forward();
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& output1);
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                         const tensor::Tensor& output1);
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                         const tensor::Tensor& input3, const tensor::Tensor& output1);
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                         const tensor::Tensor& input3, const tensor::Tensor& input4,
                         const tensor::Tensor& output1);
    base::Status forward(const tensor::Tensor& input1, const tensor::Tensor& input2,
                         const tensor::Tensor& input3, const tensor::Tensor& input4,
                         const tensor::Tensor& input5, const tensor::Tensor& output1);

    // Device and dtype must match; with dims, the shape too.
    base::Status check_tensor(const tensor::Tensor& tensor, base::DeviceType device_type,
                              base::DataType data_type) const;
    base::Status check_tensor_with_dim(const tensor::Tensor& tensor, base::DeviceType device_type,
                                       base::DataType data_type, ...) const;

    void set_input(int32_t idx, const tensor::Tensor& input);
    void set_output(int32_t idx, const tensor::Tensor& output);
    size_t inputs_size() const { return inputs_.size(); }
    size_t outputs_size() const { return outputs_.size(); }
    tensor::Tensor& get_input(int32_t idx);
    tensor::Tensor& get_output(int32_t idx);
    const tensor::Tensor& get_input(int32_t idx) const;
    const tensor::Tensor& get_output(int32_t idx) const;
    void reset_inputs_size(size_t size) { inputs_.resize(size); }
    void reset_outputs_size(size_t size) { outputs_.resize(size); }

    void set_cuda_config(std::shared_ptr<kernel::CudaConfig> cuda_config) {
        cuda_config_ = std::move(cuda_config);
    }
    std::shared_ptr<kernel::CudaConfig> cuda_config() const { return cuda_config_; }

    const std::string& layer_name() const { return layer_name_; }
    LayerType layer_type() const { return layer_type_; }
    base::DataType data_type() const { return data_type_; }
    base::DeviceType device_type() const { return device_type_; }
    void set_device_type(base::DeviceType device_type) { device_type_ = device_type; }

protected:
    base::Status bind_and_run(std::initializer_list<const tensor::Tensor*> inputs,
                              const tensor::Tensor& output);

    base::DeviceType device_type_;
    LayerType layer_type_;
    // Every operator of the reference computes in BF16 (code/source/op/layer.cpp:41-42).
    base::DataType data_type_ = base::DataType::DataTypeBf16;
    std::string layer_name_;
    std::vector<tensor::Tensor> inputs_;
    std::vector<tensor::Tensor> outputs_;
    std::shared_ptr<kernel::CudaConfig> cuda_config_;
};

class LayerParam : public Layer {
public:
    explicit LayerParam(base::DeviceType device_type, LayerType layer_type,
                        bool is_quant_layer = false, std::string layer_name = "");
    size_t weights_size() const { return weights_.size(); }
    void reset_weights_size(size_t size) { weights_.resize(size); }
    tensor::Tensor& get_weight(int32_t idx);
    const tensor::Tensor& get_weight(int32_t idx) const;
    base::Status set_weight(int32_t idx, const tensor::Tensor& weight);
    // Borrows `weight_ptr` as a tensor of shape `dims` living on `device_type`.
    base::Status set_weight(int32_t idx, const std::vector<int32_t>& dims, const void* weight_ptr,
                            base::DeviceType device_type);

protected:
    bool is_quant_layer_ = false;
    std::vector<tensor::Tensor> weights_;
};

}  // namespace op

#endif  // LLMINFER_SHIM_OP_LAYER_H
