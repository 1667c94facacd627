// QK-Norm + rotate-half RoPE of one 128-channel head by one warp, shared by the stand-alone
// front-stage kernel and by the attention kernel's fused prologue so that both give the same
// bits.
//
// Arithmetic follows fused_qk_norm_rope_kernel
// (code/source/op/kernel/cuda/rmsnorm_kernel.cu:205-244) operation for operation, including
// the shape of its sum-of-squares reduction (four 32-element shuffle trees, then
// (w0 + w2) + (w1 + w3)):
//     s  = rsqrtf(sum(x^2) / 128 + eps)
//     a  = x[i] * w[i] * s,  b = x[i + 64] * w[i + 64] * s           (FP32, no rounding)
//     y[i] = a * cos[i] - b * sin[i],  y[i + 64] = a * sin[i] + b * cos[i]   -> BF16
// Lane l owns channels l, 32 + l, 64 + l, 96 + l, i.e. the rotation pairs (l, 64 + l) and
// (32 + l, 96 + l).
#pragma once

#include <cuda_bf16.h>

namespace gqa {

__device__ __forceinline__ float front_tree_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// freq_i = 1 / powf(1e6, 2i / 128), as sin_cos_cache_kernel
// (code/source/op/kernel/cuda/rope_kernel.cu:6-21) computes it.
__device__ __forceinline__ float front_rope_freq(int i) {
    return 1.0f / powf(1000000.0f, (2.0f * i) / 128);
}

// in: the head's 128 BF16 channels; wei: its 128 norm weights; sin_row / cos_row: the 64
// angles of the token's position (null: computed from `pos`). y[0..3] are the rotated
// channels lane, lane + 32, lane + 64, lane + 96, already rounded to BF16.
__device__ __forceinline__ void front_norm_rope(const __nv_bfloat16* in, const __nv_bfloat16* wei,
                                                const float* sin_row, const float* cos_row,
                                                int32_t pos, float eps, int lane,
                                                __nv_bfloat16 (&y)[4]) {
    const float x0 = __bfloat162float(in[lane]);
    const float x1 = __bfloat162float(in[lane + 32]);
    const float x2 = __bfloat162float(in[lane + 64]);
    const float x3 = __bfloat162float(in[lane + 96]);
    const float w0 = front_tree_sum(x0 * x0);
    const float w1 = front_tree_sum(x1 * x1);
    const float w2 = front_tree_sum(x2 * x2);
    const float w3 = front_tree_sum(x3 * x3);
    const float sum = (w0 + w2) + (w1 + w3);
    const float scale = rsqrtf(sum / 128 + eps);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int pair_id = lane + half * 32;
        float sin_theta, cos_theta;
        if (sin_row != nullptr) {
            sin_theta = sin_row[pair_id];
            cos_theta = cos_row[pair_id];
        } else {
            const float theta = static_cast<float>(pos) * front_rope_freq(pair_id);
            sincosf(theta, &sin_theta, &cos_theta);
        }
        const float xa = half == 0 ? x0 : x1;
        const float xb = half == 0 ? x2 : x3;
        const float a = xa * __bfloat162float(wei[pair_id]) * scale;
        const float bb = xb * __bfloat162float(wei[pair_id + 64]) * scale;
        const float a1 = a * cos_theta - bb * sin_theta;
        const float b1 = a * sin_theta + bb * cos_theta;
        y[half] = __float2bfloat16(a1);
        y[half + 2] = __float2bfloat16(b1);
    }
}

}  // namespace gqa
