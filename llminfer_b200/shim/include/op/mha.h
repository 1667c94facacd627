// op::MultiHeadAttention of the reference (code/include/op/mha.h:7-26,
// code/source/op/mha.cpp:5-66): four inputs (query, key cache, value cache, KV-split
// scratch), one output, the position and layer set per call.
#ifndef LLMINFER_SHIM_OP_MHA_H
#define LLMINFER_SHIM_OP_MHA_H

#include "op/layer.h"

namespace op {

class MultiHeadAttention : public Layer {
public:
    explicit MultiHeadAttention(base::DeviceType device_type, int32_t kv_dim, int32_t kv_mul,
                                int32_t head_num, int32_t head_dim, int32_t max_seq_len);
    base::Status check() const override;
    base::Status forward() override;
    using Layer::forward;
    void set_pos(int32_t pos) { pos_ = pos; }
    void set_layer_id(int32_t layer_id) { layer_id_ = layer_id; }

private:
    int32_t layer_id_ = 0;
    int32_t pos_ = 0;
    int32_t kv_dim_ = 0;
    int32_t kv_mul_ = 0;
    int32_t head_num_ = 0;
    int32_t head_dim_ = 0;
    int32_t max_seq_len_ = 0;
};

}  // namespace op

#endif  // LLMINFER_SHIM_OP_MHA_H
