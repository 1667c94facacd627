// Launchers of the device kernels, called by the C ABI in gqa_api.cu.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/gqa_b200.h"
#include "work_map.cuh"

namespace gqa {

// Shape of the BF16 streaming kernel: warps per CTA (each with its own staging ring), stages
// per ring, keys per stage and CTAs resident per SM. Each CTA keeps
// warps * stages * keys * 512 bytes of K/V in flight (128 KiB per SM measured best).
struct StreamShape {
    int warps;
    int stages;
    int keys;
    int ctas_per_sm;
};
constexpr StreamShape kDefaultStreamShape = {4, 1, 64, 1};

size_t stream_bf16_smem_bytes(int warps, int stages, int keys, int n_tiles, bool fused,
                              bool cluster, int batch_for_tables);

// What the BF16 streaming kernel needs to run the front stage itself (QK-Norm + RoPE of the
// raw query rows in DecodeArgs::q, and of the new key rows, which it appends to the cache
// together with the value rows). Token t of sequence b sits at position len_b - q_tokens + t.
struct FusedFrontArgs {
    const void* k_new;      // [batch][q_tokens][num_kv_heads][128] raw keys
    const void* v_new;      // same shape
    const void* qk_weight;  // [2][128]: query norm weights, key norm weights
    void* q_out;            // optional: the rotated queries, laid out like q
    const float* sin_cache; // [table_len][64] or null (angles computed in the kernel)
    const float* cos_cache;
    int32_t table_len;
    float eps;
};

// The tensor maps must have been encoded with a box of kDefaultStreamShape.keys rows. With
// `fused` the kernel also runs the front stage (see FusedFrontArgs). group * q_tokens <= 16.
// With args.cluster_size > 0 the launch is one cluster of that many CTAs per unit (grid =
// units * cluster_size) and the splits are merged inside the clusters: no combine launch.
cudaError_t launch_stream_bf16(const CUtensorMap& tmap_k, const CUtensorMap& tmap_v,
                               const DecodeArgs& args, const FusedFrontArgs* fused, int grid,
                               cudaStream_t stream);
// Clusters of args.cluster_size CTAs of that kernel the GPU holds at once (0: none, or the
// query failed).
int stream_bf16_max_clusters(const CUtensorMap& tmap_k, const CUtensorMap& tmap_v,
                             const DecodeArgs& args, const FusedFrontArgs* fused, int grid);

cudaError_t launch_stream_f32(const DecodeArgs& args, int grid, cudaStream_t stream);

struct PeerGatherArgs;

// One CTA per output row (sequence, query token, query head); merges the partial records of
// split units.
//   kLocal   writes the finished rows of split units to DecodeArgs::out;
//   kGather  also exchanges the finished rows with the other ranks of a KV-head-parallel node
//            through the peer windows in `gather` (allowed when combine_can_gather());
//   kSeqPar  merges the row with the records the other ranks computed on their slices of the
//            keys (records travel through the peer windows in `gather`);
//   kRecord  leaves the row's record (128 channel sums, maximum, row sum) in gather->recv
//            ([rows][130] floats) instead of an output row.
enum class CombineKind { kLocal, kGather, kSeqPar, kRecord };
cudaError_t launch_combine(const DecodeArgs& args, bool bf16_out, cudaStream_t stream,
                           const PeerGatherArgs* gather = nullptr,
                           CombineKind kind = CombineKind::kLocal);
bool combine_can_gather(int rows, int sm_count);
int combine_resident_ctas(int grid, int sm_count);

// out[row] = merge of records[part][row] over the parts, in ascending order.
cudaError_t launch_merge_partials(const float* records, int32_t nparts, int64_t rows,
                                  bool bf16_out, void* out, cudaStream_t stream);

// gqa_decode with the gather fused into the combine kernel when that is possible; *fused
// tells whether it was (if not, nothing was exchanged and the caller gathers separately).
int decode_with_gather(const gqa_decode_params* p, const gqa_fused_front* front,
                       const PeerGatherArgs* gather, bool* fused);

// Sequence-parallel decode: p describes this rank's slice of every sequence (all heads); the
// combine kernel merges the ranks' records through the peer windows and writes the complete
// output on every rank.
int decode_sequence_parallel(const gqa_decode_params* p, const PeerGatherArgs* gather);

// Tensor map of a row-major BF16 matrix [rows][cols] with `pitch` elements between rows, boxes
// of 16 rows x 64 columns in 128-byte swizzled rows (cached: weights keep their address).
int cached_matrix_map(const void* base, int64_t cols, int64_t rows, int64_t pitch,
                      CUtensorMap* map);

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
    int32_t k_in_place;  // k_new already is the cache row: rotate it where it lies
    int32_t q_tokens;      // new tokens per sequence, at consecutive positions
    int32_t pos_capacity;  // positions a sequence can hold
    int32_t table_len;     // rows of the sin/cos tables
    int32_t num_blocks;    // blocks in the cache
    int32_t* status;       // raised when a device-side position or block id is out of range
    float eps;
};

cudaError_t launch_front(const FrontArgs& args, cudaStream_t stream);

// Launches `kernel` so that it may start while the preceding kernel of the stream is still
// running (programmatic dependent launch). Such a kernel calls pdl_wait() before it touches
// anything an earlier kernel wrote, and everything before that call overlaps the
// predecessor's tail and the launch latency.
template <typename... KernelArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                       cudaStream_t stream, Args&&... args) {
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KernelArgs>(args)...);
}

cudaError_t launch_sin_cos(float* sin_cache, float* cos_cache, int32_t head_dim,
                           int32_t max_seq_len, cudaStream_t stream);

}  // namespace gqa
