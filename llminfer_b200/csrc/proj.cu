// Output projection with residual add behind decode attention; see include/gqa_b200.h.
//
// Takes the place of fused_gemv_add_bf16x8_kernel
// (code/source/op/kernel/cuda/matmul_kernel.cu:143-170): residual[n] += dot(x, W[n]). There one
// CTA of 256 threads owns one output row of one token. Here the weights are streamed once for
// up to 8 tokens and multiplied on tensor cores: a warp owns 16 weight rows (the M side of
// mma.m16n8k16), the tokens sit on the N side, accumulation is FP32.
//
// Fragments come straight from global memory, without a shared-memory stage: a dot product
// does not care in which order its terms are added, so within a block of 32 columns thread
// (g, t) of a warp loads the 8 consecutive columns 8t..8t+7 of rows g and g+8 with two 16-byte
// loads, takes the same 8 columns of token g's activations, and feeds them to two MMAs as if
// they were the columns the fragment layout expects. Both operands use the same permutation,
// every column is used exactly once.
//
// Summation order (fixed, so that a KV-head-parallel node reproduces the single-GPU result
// bit for bit): one partial per query head (128 columns, 8 MMAs from a zero accumulator),
// heads added in ascending order per KV head, KV heads added in ascending order, then the
// residual. A CTA of 8 warps covers 16 * tiles_per_cta rows and all local heads; head partials
// meet in shared memory. In the sharded form every rank pushes its per-KV-head sums to the
// peers' windows as step-tagged words (plain stores over NVLink) and polls, with a time
// limit, for the sums of the KV heads it does not own.
#include "../../include/gqa_b200.h"

#include <cstring>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "decode_kernels.cuh"
#include "peer_window.cuh"
#include "ptx.cuh"

namespace gqa {
namespace {

constexpr int kProjWarps = 8;
constexpr int kProjThreads = kProjWarps * 32;
constexpr int kProjTokens = 8;   // tokens per launch: the N side of the MMA
constexpr int kTileRows = 16;    // weight rows per warp: the M side of the MMA
constexpr int kTileOutputs = kTileRows * kProjTokens;
constexpr int kMaxLocalGroups = 8;

struct OprojArgs {
    const __nv_bfloat16* x;    // [batch][heads * 128]
    const __nv_bfloat16* w;    // row n, column c at w[n * ld + c]
    __nv_bfloat16* residual;   // [batch][hidden]
    int64_t ld;
    int32_t batch;             // <= 8
    int32_t hidden;
    int32_t heads;             // local query heads
    int32_t groups;            // local KV heads
    int32_t tiles_per_cta;
    int32_t heads_per_warp;
};

template <bool SHARDED>
__global__ void __launch_bounds__(kProjThreads, 3)
    oproj_residual_kernel(const OprojArgs a, const PeerGatherArgs g) {
    extern __shared__ float s_part[];  // [tiles_per_cta][heads][16 rows][8 tokens]
    __shared__ uint32_t s_step;
    __shared__ int s_timed_out;
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int gid = lane >> 2;
    const int tig = lane & 3;
    const int warps_per_tile = kProjWarps / a.tiles_per_cta;
    const int tile_in_cta = warp / warps_per_tile;
    // Warp `sub` of a tile takes heads sub, sub + warps_per_tile, ...: at any moment the warps
    // of a tile read neighbouring 256-byte pieces of the same weight rows.
    const int sub = warp - tile_in_cta * warps_per_tile;
    const int row0 = (blockIdx.x * a.tiles_per_cta + tile_in_cta) * kTileRows;
    const bool active = row0 < a.hidden;
    const int xcols = a.heads * kHeadDim;

    uint4 wlo[4], whi[4];
    const __nv_bfloat16* wrow = a.w + (int64_t)(row0 + gid) * a.ld + sub * kHeadDim + 8 * tig;
    auto load_weights = [&](int hh) {
        const __nv_bfloat16* p = wrow + (int64_t)hh * warps_per_tile * kHeadDim;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            wlo[kb] = __ldcs(reinterpret_cast<const uint4*>(p + 32 * kb));
            whi[kb] = __ldcs(reinterpret_cast<const uint4*>(p + 8 * a.ld + 32 * kb));
        }
    };
    // The weights do not depend on the kernel in front: fetch the first head's before waiting.
    if (active) load_weights(0);
    pdl_wait();
    if (SHARDED && threadIdx.x == 0) {
        WindowCtrl* ctrl = window_ctrl(g.windows[g.rank], g.slot_bytes, g.nranks);
        s_step = *reinterpret_cast<volatile uint32_t*>(&ctrl->step) + 1;
        s_timed_out = 0;
    }
    if (active) {
        for (int hh = 0; hh < a.heads_per_warp; ++hh) {
            const int head = hh * warps_per_tile + sub;
            uint4 xf[4];
            if (gid < a.batch) {
                const __nv_bfloat16* xp = a.x + (int64_t)gid * xcols + head * kHeadDim + 8 * tig;
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) {
                    xf[kb] = __ldcg(reinterpret_cast<const uint4*>(xp + 32 * kb));
                }
            } else {
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) xf[kb] = make_uint4(0u, 0u, 0u, 0u);
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                mma_bf16_16816(acc, wlo[kb].x, whi[kb].x, wlo[kb].y, whi[kb].y, xf[kb].x, xf[kb].y);
                mma_bf16_16816(acc, wlo[kb].z, whi[kb].z, wlo[kb].w, whi[kb].w, xf[kb].z, xf[kb].w);
            }
            if (hh + 1 < a.heads_per_warp) load_weights(hh + 1);
            float* dst = s_part + (int64_t)(tile_in_cta * a.heads + head) * kTileOutputs;
            *reinterpret_cast<float2*>(dst + gid * kProjTokens + 2 * tig) =
                make_float2(acc[0], acc[1]);
            *reinterpret_cast<float2*>(dst + (gid + 8) * kProjTokens + 2 * tig) =
                make_float2(acc[2], acc[3]);
        }
    }
    __syncthreads();

    // One thread per (tile, token, row) at a time: heads -> KV-head sums -> total -> residual.
    bool timed_out = false;
    for (int o = threadIdx.x; o < a.tiles_per_cta * kTileOutputs; o += kProjThreads) {
        const int t = o >> 7;
        const int b = (o & 127) >> 4;
        const int n = (blockIdx.x * a.tiles_per_cta + t) * kTileRows + (o & 15);
        if (b >= a.batch || n >= a.hidden || timed_out) continue;
        const float* part =
            s_part + (int64_t)t * a.heads * kTileOutputs + (o & 15) * kProjTokens + b;
        const int per_group = a.heads / a.groups;
        float sums[kMaxLocalGroups];
#pragma unroll
        for (int lg = 0; lg < kMaxLocalGroups; ++lg) {
            sums[lg] = 0.f;
            if (lg < a.groups) {
                const float* p = part + (int64_t)lg * per_group * kTileOutputs;
                float s = p[0];
                for (int j = 1; j < per_group; ++j) s += p[j * kTileOutputs];
                sums[lg] = s;
            }
        }
        float total = 0.f;
        if (!SHARDED) {
#pragma unroll
            for (int lg = 0; lg < kMaxLocalGroups; ++lg) {
                if (lg < a.groups) total += sums[lg];
            }
        } else {
            const uint32_t step = s_step;
            const uint64_t per_token = (uint64_t)a.hidden;
#pragma unroll
            for (int lg = 0; lg < kMaxLocalGroups; ++lg) {
                if (lg < a.groups) {
                    const uint64_t word = ((uint64_t)lg * a.batch + b) * per_token + n;
                    for (int p = 0; p < g.nranks; ++p) {
                        if (p == g.rank) continue;
                        push_word(window_slot(g.windows[p], step, g.nranks, g.rank, g.slot_bytes) +
                                      word,
                                  step, __float_as_uint(sums[lg]));
                    }
                }
            }
            const unsigned long long start = global_timer();
            uint8_t* mine = g.windows[g.rank];
            for (int r = 0; r < g.nranks && !timed_out; ++r) {
#pragma unroll
                for (int lg = 0; lg < kMaxLocalGroups; ++lg) {
                    if (lg < a.groups && !timed_out) {
                        float v = sums[lg];
                        if (r != g.rank) {
                            const uint64_t word = ((uint64_t)lg * a.batch + b) * per_token + n;
                            uint32_t bits = 0;
                            if (poll_word(window_slot(mine, step, g.nranks, r, g.slot_bytes) + word,
                                          step, start, &bits)) {
                                v = __uint_as_float(bits);
                            } else {
                                timed_out = true;
                            }
                        }
                        total += v;
                    }
                }
            }
        }
        if (!timed_out) {
            __nv_bfloat16* out = a.residual + (int64_t)b * a.hidden + n;
            *out = __float2bfloat16(__bfloat162float(*out) + total);
        }
    }
    if (SHARDED) {
        if (timed_out) s_timed_out = 1;
        __syncthreads();
        if (threadIdx.x == 0) {
            WindowCtrl* ctrl = window_ctrl(g.windows[g.rank], g.slot_bytes, g.nranks);
            if (s_timed_out) {
                ctrl->status = 1;
                if (g.status != nullptr) atomicExch(g.status, 2);
            }
            // The last CTA to finish advances the step counter for the next launch.
            __threadfence();
            const uint32_t ticket = atomicAdd(&ctrl->ticket_out, 1u);
            if (ticket == gridDim.x - 1) {
                ctrl->ticket_out = 0;
                ctrl->step = s_step;
            }
        }
    }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int validate(const gqa_oproj_params* p, int* tiles_per_cta, int* heads_per_warp) {
    if (p == nullptr) return GQA_ERR_NULL;
    if (p->attn_out == nullptr || p->weight == nullptr || p->residual == nullptr) {
        return GQA_ERR_NULL;
    }
    if (p->head_dim != kHeadDim || p->batch <= 0 || p->hidden <= 0 || p->hidden % kTileRows != 0) {
        return GQA_ERR_SHAPE;
    }
    const int heads = p->num_q_heads;
    if (heads <= 0 || p->num_kv_heads <= 0 || p->num_kv_heads > kMaxLocalGroups ||
        heads % p->num_kv_heads != 0) {
        return GQA_ERR_SHAPE;
    }
    if (heads % kProjWarps == 0) {
        *tiles_per_cta = 1;
        *heads_per_warp = heads / kProjWarps;
    } else if (heads == 1 || heads == 2 || heads == 4) {
        *tiles_per_cta = kProjWarps / heads;
        *heads_per_warp = 1;
    } else {
        return GQA_ERR_SHAPE;
    }
    if ((size_t)*tiles_per_cta * heads * kTileOutputs * sizeof(float) > 48 * 1024) {
        return GQA_ERR_SHAPE;
    }
    if (p->weight_ld < (int64_t)heads * kHeadDim || p->weight_ld % 8 != 0) return GQA_ERR_SHAPE;
    if (!aligned16(p->attn_out) || !aligned16(p->weight)) return GQA_ERR_ALIGN;
    return GQA_OK;
}

int run(const gqa_oproj_params* p, gqa_comm* comm) {
    int tiles_per_cta = 0, heads_per_warp = 0;
    const int rc = validate(p, &tiles_per_cta, &heads_per_warp);
    if (rc != GQA_OK) return rc;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(p->stream);
    const int tiles = p->hidden / kTileRows;
    const int grid = (tiles + tiles_per_cta - 1) / tiles_per_cta;
    const size_t smem = (size_t)tiles_per_cta * p->num_q_heads * kTileOutputs * sizeof(float);
    // More than 8 tokens: one pass over the weights per 8 (each its own exchange step).
    for (int b0 = 0; b0 < p->batch; b0 += kProjTokens) {
        OprojArgs a;
        std::memset(&a, 0, sizeof(a));
        a.batch = p->batch - b0 < kProjTokens ? p->batch - b0 : kProjTokens;
        a.x = static_cast<const __nv_bfloat16*>(p->attn_out) +
              (int64_t)b0 * p->num_q_heads * kHeadDim;
        a.w = static_cast<const __nv_bfloat16*>(p->weight);
        a.residual = static_cast<__nv_bfloat16*>(p->residual) + (int64_t)b0 * p->hidden;
        a.ld = p->weight_ld;
        a.hidden = p->hidden;
        a.heads = p->num_q_heads;
        a.groups = p->num_kv_heads;
        a.tiles_per_cta = tiles_per_cta;
        a.heads_per_warp = heads_per_warp;
        PeerGatherArgs g;
        std::memset(&g, 0, sizeof(g));
        cudaError_t e;
        if (comm != nullptr && gqa_comm_nranks(comm) > 1) {
            const size_t bytes = (size_t)p->num_kv_heads * a.batch * p->hidden * sizeof(float);
            const int crc = comm_peer_args(comm, bytes, p->status_dev, &g);
            if (crc != GQA_OK) return crc;
            e = launch_pdl(oproj_residual_kernel<true>, dim3(grid), dim3(kProjThreads), smem,
                           stream, a, g);
        } else {
            e = launch_pdl(oproj_residual_kernel<false>, dim3(grid), dim3(kProjThreads), smem,
                           stream, a, g);
        }
        if (e != cudaSuccess) return GQA_ERR_CUDA;
    }
    return GQA_OK;
}

}  // namespace
}  // namespace gqa

extern "C" {

int gqa_oproj_residual(const gqa_oproj_params* p) { return gqa::run(p, nullptr); }

int gqa_oproj_residual_sharded(const gqa_oproj_params* p, gqa_comm* comm) {
    if (comm == nullptr) return GQA_ERR_NULL;
    return gqa::run(p, comm);
}

}  // extern "C"
