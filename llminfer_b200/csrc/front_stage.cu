// Front stage of decode attention: per-head RMSNorm (QK-Norm) + rotate-half RoPE on the new
// tokens' queries and keys, with the key and value rows appended to the KV cache in the same
// launch; and the sin/cos table builder.
//
// The arithmetic (front_math.cuh) follows fused_qk_norm_rope_kernel
// (code/source/op/kernel/cuda/rmsnorm_kernel.cu:205-244) operation for operation, so that
// results can agree with it bit for bit. One warp handles one head.
//
// The table builder follows sin_cos_cache_kernel (code/source/op/kernel/cuda/rope_kernel.cu:6-21).
#include <cuda_bf16.h>

#include "decode_kernels.cuh"
#include "front_math.cuh"
#include "ptx.cuh"

namespace gqa {

namespace {

constexpr int kFrontWarps = 4;

// blockIdx.y = sequence * q_tokens + token: token t of sequence b sits at position pos_b + t.
__global__ void __launch_bounds__(kFrontWarps * 32) qk_norm_rope_append_kernel(const FrontArgs f) {
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bt = blockIdx.y;
    const int b = bt / f.q_tokens;
    const int row = blockIdx.x * kFrontWarps + warp;
    const int n_rows = f.num_q_heads + (f.v_new != nullptr ? 2 : 1) * f.num_kv_heads;
    pdl_launch_dependents();
    pdl_wait();
    if (row >= n_rows) return;

    const int32_t pos =
        (f.positions_dev != nullptr ? f.positions_dev[b] : f.uniform_pos) + (bt - b * f.q_tokens);
    // A position read from device memory decides where rows are WRITTEN: one that lies outside
    // the cache (or the angle table) skips the row and raises the status word.
    bool ok = pos >= 0 && pos < f.pos_capacity && (f.sin_cache == nullptr || pos < f.table_len);
    int32_t blk = f.fixed_block;
    int32_t tok = pos;
    if (ok && f.block_table != nullptr && !f.k_in_place) {
        const int32_t lb = pos / f.block_tokens;
        tok = pos - lb * f.block_tokens;
        blk = f.block_table[(int64_t)b * f.blocks_per_seq + lb];
        ok = blk >= 0 && blk < f.num_blocks;
    }
    if (!ok) {
        if (lane == 0 && f.status != nullptr) atomicExch(f.status, kStatusBadInput);
        return;
    }
    // Cache row of this token for kv head `hk`.
    auto cache_off = [&](int hk) -> int64_t {
        return (int64_t)blk * f.stride_block + (int64_t)tok * f.stride_token +
               (int64_t)hk * f.stride_head;
    };

    if (row >= f.num_q_heads + f.num_kv_heads) {
        // Value row: stored as it is.
        const int hk = row - f.num_q_heads - f.num_kv_heads;
        const uint2* src = reinterpret_cast<const uint2*>(
            reinterpret_cast<const __nv_bfloat16*>(f.v_new) +
            ((int64_t)bt * f.num_kv_heads + hk) * kHeadDim);
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
        const int64_t off = ((int64_t)bt * f.num_q_heads + row) * kHeadDim;
        in = reinterpret_cast<const __nv_bfloat16*>(f.q) + off;
        out = reinterpret_cast<__nv_bfloat16*>(f.q_out) + off;
    } else {
        const int hk = row - f.num_q_heads;
        in = reinterpret_cast<const __nv_bfloat16*>(f.k_new) +
             ((int64_t)bt * f.num_kv_heads + hk) * kHeadDim;
        out = f.k_in_place ? const_cast<__nv_bfloat16*>(in)
                           : reinterpret_cast<__nv_bfloat16*>(f.k_cache) + cache_off(hk);
        wei += kHeadDim;
    }
    const float* sin_row = f.sin_cache != nullptr ? f.sin_cache + (int64_t)pos * (kHeadDim / 2) : nullptr;
    const float* cos_row = f.cos_cache != nullptr ? f.cos_cache + (int64_t)pos * (kHeadDim / 2) : nullptr;
    __nv_bfloat16 y[4];
    front_norm_rope(in, wei, sin_row, cos_row, pos, f.eps, lane, y);
#pragma unroll
    for (int i = 0; i < 4; ++i) out[lane + 32 * i] = y[i];
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
    dim3 grid((n_rows + kFrontWarps - 1) / kFrontWarps, args.batch * args.q_tokens);
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
