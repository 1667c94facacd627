// op::QKNormRoPELaryer of the reference (code/include/op/qk_norm_rope.h,
// code/source/op/qk_norm_rope.cpp:5-70; the class name keeps the reference's spelling): five
// inputs (query, key row, token position on the CPU, sin table, cos table) and one weight
// [2 * head_dim] = q_norm then k_norm.
#ifndef LLMINFER_SHIM_OP_QK_NORM_ROPE_H
#define LLMINFER_SHIM_OP_QK_NORM_ROPE_H

#include "op/layer.h"

namespace op {

class QKNormRoPELaryer : public LayerParam {
public:
    explicit QKNormRoPELaryer(base::DeviceType device_type, int32_t dim, int32_t kv_dim,
                              int32_t head_dim);
    base::Status check() const override;
    base::Status forward() override;
    using Layer::forward;

private:
    int32_t dim_ = 0;
    int32_t kv_dim_ = 0;
    int32_t head_dim_ = 0;
};

}  // namespace op

#endif  // LLMINFER_SHIM_OP_QK_NORM_ROPE_H
