// Launchers of the device kernels, called by the C ABI in gqa_api.cu.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "work_map.cuh"

namespace gqa {

// Shape of the BF16 streaming kernel: warps per CTA (each with its own staging ring) and
// stages per ring. 4 x 3 x 16 KiB = 192 KiB of K/V in flight per SM.
constexpr int kStreamWarps = 4;
constexpr int kStreamStages = 3;

size_t stream_bf16_smem_bytes(int warps, int stages, int batch_for_tables);

cudaError_t launch_stream_bf16(const CUtensorMap& tmap_k, const CUtensorMap& tmap_v,
                               const DecodeArgs& args, int grid, cudaStream_t stream);

cudaError_t launch_stream_f32(const DecodeArgs& args, int grid, cudaStream_t stream);

// One CTA per (sequence, query head); merges the partial records of split units.
cudaError_t launch_combine(const DecodeArgs& args, bool bf16_out, cudaStream_t stream);

struct FrontArgs {
    const void* q;
    void* q_out;
    const void* k_new;
    const void* v_new;
    const void* qk_weight;
    void* k_cache;
    void* v_cache;
    const float* sin_cache;
    const float* cos_cache;
    const int32_t* positions_dev;
    const int32_t* block_table;
    int64_t stride_block;
    int64_t stride_token;
    int64_t stride_head;
    int32_t batch;
    int32_t num_q_heads;
    int32_t num_kv_heads;
    int32_t uniform_pos;
    int32_t blocks_per_seq;
    int32_t block_tokens;
    int32_t fixed_block;
    float eps;
};

cudaError_t launch_front(const FrontArgs& args, cudaStream_t stream);

cudaError_t launch_sin_cos(float* sin_cache, float* cos_cache, int32_t head_dim,
                           int32_t max_seq_len, cudaStream_t stream);

}  // namespace gqa
