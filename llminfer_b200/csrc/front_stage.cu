// Front stage of decode attention: per-head RMSNorm (QK-Norm) + rotate-half RoPE on the new
// token's query and key, with the key and value rows appended to the KV cache in the same
// launch; and the sin/cos table builder.
//
// Arithmetic follows fused_qk_norm_rope_kernel
// (code/source/op/kernel/cuda/rmsnorm_kernel.cu:205-244) operation for operation, including
// the shape of its sum-of-squares reduction (four 32-element shuffle trees, then
// (w0 + w2) + (w1 + w3)), so that results can agree with it bit for bit:
//     s  = rsqrtf(sum(x^2) / 128 + eps)
//     a  = x[i] * w[i] * s,  b = x[i + 64] * w[i + 64] * s           (FP32, no rounding)
//     y[i] = a * cos[i] - b * sin[i],  y[i + 64] = a * sin[i] + b * cos[i]   -> BF16
// One warp handles one head; lane l owns channels l, 32 + l, 64 + l, 96 + l, i.e. the two
// rotation pairs (l, 64 + l) and (32 + l, 96 + l).
//
// The table builder follows sin_cos_cache_kernel (code/source/op/kernel/cuda/rope_kernel.cu:6-21).
#include <cuda_bf16.h>

#include "decode_kernels.cuh"
#include "ptx.cuh"

namespace gqa {

namespace {

constexpr int kFrontWarps = 4;

__device__ __forceinline__ float tree_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

__device__ __forceinline__ float rope_freq(int i) {
    return 1.0f / powf(1000000.0f, (2.0f * i) / kHeadDim);
}

__global__ void __launch_bounds__(kFrontWarps * 32) qk_norm_rope_append_kernel(const FrontArgs f) {
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.y;
    const int row = blockIdx.x * kFrontWarps + warp;
    const int n_rows = f.num_q_heads + (f.v_new != nullptr ? 2 : 1) * f.num_kv_heads;
    pdl_launch_dependents();
    pdl_wait();
    if (row >= n_rows) return;

    const int32_t pos = f.positions_dev != nullptr ? f.positions_dev[b] : f.uniform_pos;

    // Cache row of this token for kv head `hk`.
    auto cache_off = [&](int hk) -> int64_t {
        int32_t blk = f.fixed_block;
        int32_t tok = pos;
        if (f.block_table != nullptr) {
            const int32_t lb = pos / f.block_tokens;
            tok = pos - lb * f.block_tokens;
            blk = f.block_table[(int64_t)b * f.blocks_per_seq + lb];
        }
        return (int64_t)blk * f.stride_block + (int64_t)tok * f.stride_token +
               (int64_t)hk * f.stride_head;
    };

    if (row >= f.num_q_heads + f.num_kv_heads) {
        // Value row: stored as it is.
        const int hk = row - f.num_q_heads - f.num_kv_heads;
        const uint2* src = reinterpret_cast<const uint2*>(
            reinterpret_cast<const __nv_bfloat16*>(f.v_new) +
            ((int64_t)b * f.num_kv_heads + hk) * kHeadDim);
        uint2* dst = reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(f.v_cache) +
                                              cache_off(hk));
        dst[lane] = src[lane];
        return;
    }

    const bool is_q = row < f.num_q_heads;
    const __nv_bfloat16* in;
    __nv_bfloat16* out;
    const __nv_bfloat16* wei = reinterpret_cast<const __nv_bfloat16*>(f.qk_weight);
    if (is_q) {
        const int64_t off = ((int64_t)b * f.num_q_heads + row) * kHeadDim;
        in = reinterpret_cast<const __nv_bfloat16*>(f.q) + off;
        out = reinterpret_cast<__nv_bfloat16*>(f.q_out) + off;
    } else {
        const int hk = row - f.num_q_heads;
        in = reinterpret_cast<const __nv_bfloat16*>(f.k_new) +
             ((int64_t)b * f.num_kv_heads + hk) * kHeadDim;
        out = f.k_in_place ? const_cast<__nv_bfloat16*>(in)
                           : reinterpret_cast<__nv_bfloat16*>(f.k_cache) + cache_off(hk);
        wei += kHeadDim;
    }

    const float x0 = __bfloat162float(in[lane]);
    const float x1 = __bfloat162float(in[lane + 32]);
    const float x2 = __bfloat162float(in[lane + 64]);
    const float x3 = __bfloat162float(in[lane + 96]);
    const float w0 = tree_sum(x0 * x0);
    const float w1 = tree_sum(x1 * x1);
    const float w2 = tree_sum(x2 * x2);
    const float w3 = tree_sum(x3 * x3);
    const float sum = (w0 + w2) + (w1 + w3);
    const float scale = rsqrtf(sum / kHeadDim + f.eps);

#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int pair_id = lane + half * 32;
        float sin_theta, cos_theta;
        if (f.sin_cache != nullptr) {
            sin_theta = f.sin_cache[(int64_t)pos * (kHeadDim / 2) + pair_id];
            cos_theta = f.cos_cache[(int64_t)pos * (kHeadDim / 2) + pair_id];
        } else {
            const float theta = static_cast<float>(pos) * rope_freq(pair_id);
            sincosf(theta, &sin_theta, &cos_theta);
        }
        const float xa = half == 0 ? x0 : x1;
        const float xb = half == 0 ? x2 : x3;
        float a = xa * __bfloat162float(wei[pair_id]) * scale;
        float bb = xb * __bfloat162float(wei[pair_id + 64]) * scale;
        float a1 = a * cos_theta - bb * sin_theta;
        float b1 = a * sin_theta + bb * cos_theta;
        out[pair_id] = __float2bfloat16(a1);
        out[pair_id + 64] = __float2bfloat16(b1);
    }
}

__global__ void sin_cos_table_kernel(float* __restrict__ sin_cache, float* __restrict__ cos_cache,
                                     int32_t half_dim, int32_t head_dim, int32_t max_seq_len) {
    const int i = blockIdx.x;
    const float freq = 1.0f / powf(1000000.0f, (2.0f * i) / head_dim);
    for (int32_t pos = blockIdx.y * blockDim.x + threadIdx.x; pos < max_seq_len;
         pos += gridDim.y * blockDim.x) {
        const float theta = static_cast<float>(pos) * freq;
        sincosf(theta, sin_cache + (int64_t)pos * half_dim + i,
                cos_cache + (int64_t)pos * half_dim + i);
    }
}

}  // namespace

cudaError_t launch_front(const FrontArgs& args, cudaStream_t stream) {
    const int n_rows = args.num_q_heads + (args.v_new != nullptr ? 2 : 1) * args.num_kv_heads;
    dim3 grid((n_rows + kFrontWarps - 1) / kFrontWarps, args.batch);
    return launch_pdl(qk_norm_rope_append_kernel, grid, dim3(kFrontWarps * 32), 0, stream, args);
}

cudaError_t launch_sin_cos(float* sin_cache, float* cos_cache, int32_t head_dim,
                           int32_t max_seq_len, cudaStream_t stream) {
    const int threads = 256;
    int slices = (max_seq_len + threads * 8 - 1) / (threads * 8);
    if (slices < 1) slices = 1;
    if (slices > 64) slices = 64;
    dim3 grid(head_dim / 2, slices);
    sin_cos_table_kernel<<<grid, threads, 0, stream>>>(sin_cache, cos_cache, head_dim / 2,
                                                        head_dim, max_seq_len);
    return cudaGetLastError();
}

}  // namespace gqa
