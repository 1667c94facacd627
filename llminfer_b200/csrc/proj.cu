// The projections on either side of decode attention: output projection with residual add
// behind it, packed QKV projection in front of it (one kernel); see include/gqa_b200.h.
//
// Takes the place of fused_gemv_add_bf16x8_kernel
// (code/source/op/kernel/cuda/matmul_kernel.cu:143-170): residual[n] += dot(x, W[n]). There one
// CTA of 256 threads owns one output row of one token. Here the weights are streamed once for
// up to 8 tokens and multiplied on tensor cores: a warp owns 16 weight rows (the M side of
// mma.m16n8k16), the tokens sit on the N side, accumulation is FP32.
//
// Work decomposition: a task is a (16-row tile, KV head) pair and belongs to one warp, which
// multiplies the KV head's columns with 8 MMAs per query head into eight independent
// accumulators. The weights arrive by TMA, one query head (16 x 128, 4 KiB, two
// boxes of 64 columns in 128-byte swizzled rows) per stage of a ring that is private to the
// warp; the warp refills a stage as soon as it has read it, so its loads run `stages` heads
// ahead of the arithmetic. Warps never wait for one another while they stream: a CTA is a
// bundle of up to four such warps that share one KV head, whose activations (up to 8 tokens)
// sit in shared memory as the B operand. A fragments come from the ring with ldmatrix.
//
// Summation order (fixed, so that a KV-head-parallel node reproduces the single-GPU result
// bit for bit): a KV head with an even number of query heads is summed in two halves (lower
// heads, upper heads), one with an odd number in one piece; per piece eight FP32 accumulators,
// one per block of 16 columns inside a query head, each running over the piece's heads in
// ascending order; the eight are added in ascending order, then lower + upper; KV heads are
// added in ascending order, then the residual.
//
// A KV head's sum is stored in a small workspace as an 8-byte word that carries the sum and
// the launch number (so no fence or atomic is needed), and in the sharded form pushed to
// every rank's window in the same format (plain stores over NVLink). The words of one
// (KV head, 16-row tile) lie together, token-major: a warp first turns its accumulator
// fragment into that order through shared memory and then stores runs of 256 bytes, instead
// of the 64-byte pieces the fragment layout would give (which cost most of the exchange at
// eight ranks). When a CTA has streamed
// all its tasks it finishes its share of the outputs: it polls (with a time limit) for the
// words of all KV heads, adds them in ascending order and updates the residual.
#include "../../include/gqa_b200.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "decode_kernels.cuh"
#include "peer_window.cuh"
#include "ptx.cuh"

namespace gqa {
namespace {

constexpr int kProjMaxWarps = 4;
constexpr int kProjTokens = 8;   // tokens per launch: the N side of the MMA
constexpr int kTileRows = 16;    // weight rows per task: the M side of the MMA
constexpr int kMaxHeadsPerGroup = 16;
constexpr int kHeadTileBytes = kTileRows * kHeadDim * 2;  // 4 KiB: one head of one tile
constexpr int kBoxBytes = kHeadTileBytes / 2;
constexpr uint64_t kProjWaitNs = 2000000000ull;
constexpr int kMaxSmem = 220 * 1024;  // leaves room for the static part (about 4 KiB)

struct OprojArgs {
    const __nv_bfloat16* x;    // [batch][heads * 128]
    __nv_bfloat16* residual;   // [batch][hidden], read and written (null in split mode)
    __nv_bfloat16* q_out;      // split mode: rows [0, q_rows) -> q_out [batch][q_rows],
    __nv_bfloat16* k_out;      // the next kv_rows rows -> k_out [batch][kv_rows],
    __nv_bfloat16* v_out;      // the last kv_rows rows -> v_out [batch][kv_rows]
    int32_t q_rows;
    int32_t kv_rows;
    WindowCtrl* ctrl;          // launch counter of the workspace (null for one KV head)
    unsigned long long* words; // [groups][batch][hidden] tagged KV-head sums
    int32_t* status;
    int32_t batch;             // <= 8
    int32_t hidden;
    int32_t heads;             // local query heads
    int32_t groups;            // local KV heads; the grid is a multiple of it
    int32_t stages;            // ring depth per warp
    int32_t team;              // warps that share a task: 1, or 2 (each streams half the heads)
};

// Waits for a stage to fill; false when the time limit ran out. The clock is looked at only
// now and then: reading it goes through the same queue as the loads and stores.
__device__ __forceinline__ bool wait_full(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long start = 0;
    for (uint32_t tries = 1;; ++tries) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((tries & 255u) == 0) {
            const unsigned long long now = global_timer();
            if (start == 0) start = now;
            if (now - start > kProjWaitNs) return false;
        }
    }
}

// Place of the sum of (KV head g, token b, output row n) among the tagged words.
__device__ __forceinline__ int64_t word_index(const OprojArgs& a, int g, int b, int n) {
    return ((((int64_t)g * (a.hidden / kTileRows) + (n / kTileRows)) * a.batch + b) * kTileRows) +
           (n % kTileRows);
}

// Where output row n of token b goes, and whether the old value is added (the residual form).
__device__ __forceinline__ __nv_bfloat16* output_at(const OprojArgs& a, int b, int n) {
    if (a.residual != nullptr) return a.residual + (int64_t)b * a.hidden + n;
    if (n < a.q_rows) return a.q_out + (int64_t)b * a.q_rows + n;
    n -= a.q_rows;
    if (n < a.kv_rows) return a.k_out + (int64_t)b * a.kv_rows + n;
    return a.v_out + (int64_t)b * a.kv_rows + (n - a.kv_rows);
}

template <bool SHARDED>
__global__ void __launch_bounds__(kProjMaxWarps * 32, 3)
    oproj_residual_kernel(const __grid_constant__ CUtensorMap wmap, const OprojArgs a,
                          const PeerGatherArgs g) {
    // [warps][stages] head tiles (1 KiB aligned), then the KV head's activations
    // [8 tokens][heads per KV head * 128 + 8] (rows padded by 16 bytes: conflict-free
    // ldmatrix), then the stage barriers.
    extern __shared__ uint8_t s_raw[];
    uint8_t* s_dyn = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(s_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ uint32_t s_step;
    __shared__ uint32_t s_local_step;
    __shared__ int s_timed_out;
    __shared__ float s_stage[kProjMaxWarps][kProjTokens * kTileRows];
    __shared__ float s_team[kProjMaxWarps / 2][2][32 * 4];
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int per_group = a.heads / a.groups;
    const int tiles = a.hidden / kTileRows;
    // CTA c works on KV head c % groups; the teams of all CTAs of a KV head share its tiles.
    // A team is one warp, or two warps that each stream half of the KV head's query heads.
    const int lg = blockIdx.x % a.groups;
    const int team = a.team;
    const int member = warp % team;
    const int unit = warp / team;
    const int units = nwarps / team;
    const int worker = (blockIdx.x / a.groups) * units + unit;
    const int workers = (gridDim.x / a.groups) * units;
    const int team_heads = per_group / team;
    const int head0 = member * team_heads;
    const int x_pitch = per_group * kHeadDim * 2 + 16;  // bytes per token row
    const uint32_t ring = smem_u32(s_dyn) + warp * a.stages * kHeadTileBytes;
    uint8_t* s_x = s_dyn + nwarps * a.stages * kHeadTileBytes;
    const uint32_t bars = smem_u32(s_x + kProjTokens * x_pitch) + warp * a.stages * 8;

    // ---- producer side: the warp's sequence of (tile, head) stages ------------------------
    const uint64_t policy = l2_policy_evict_first();
    int prod_tile = worker, prod_head = head0, prod_stage = 0;
    auto issue = [&]() {
        if (prod_tile >= tiles) return;
        if (lane == 0) {
            const int col = (lg * per_group + prod_head) * kHeadDim;
            const uint32_t bar = bars + prod_stage * 8;
            const uint32_t dst = ring + prod_stage * kHeadTileBytes;
            // No proxy fence: the stage was only read, and every lane's ldmatrix results had
            // been consumed by its MMAs before the __syncwarp that precedes this call.
            mbar_arrive_expect_tx(bar, kHeadTileBytes);
            tma_load_2d(dst, &wmap, bar, col, prod_tile * kTileRows, policy);
            tma_load_2d(dst + kBoxBytes, &wmap, bar, col + 64, prod_tile * kTileRows, policy);
        }
        if (++prod_stage == a.stages) prod_stage = 0;
        if (++prod_head == head0 + team_heads) {
            prod_head = head0;
            prod_tile += workers;
        }
    };
    if (lane == 0) {
        prefetch_tensormap(&wmap);
        for (int s = 0; s < a.stages; ++s) mbar_init(bars + s * 8, 1);
        mbar_init_fence();
    }
    __syncwarp();
    // The weights do not depend on the kernel in front: fill the ring before waiting for it.
    for (int s = 0; s < a.stages; ++s) issue();
    pdl_wait();
    if (threadIdx.x == 0) {
        s_timed_out = 0;
        s_step = 0;
        s_local_step = 0;
        if (SHARDED) {
            WindowCtrl* ctrl = window_ctrl(g.windows[g.rank], g.slot_bytes, g.nranks);
            s_step = *reinterpret_cast<volatile uint32_t*>(&ctrl->step) + 1;
        }
        if (a.ctrl != nullptr) {
            s_local_step = *reinterpret_cast<volatile uint32_t*>(&a.ctrl->step) + 1;
        }
    }
    {
        // The KV head's activations, tokens beyond the batch as zeros.
        const int per_token = per_group * (kHeadDim / 8);
        const int xcols = a.heads * kHeadDim;
        for (int i = threadIdx.x; i < kProjTokens * per_token; i += blockDim.x) {
            const int tok = i / per_token;
            const int c = i - tok * per_token;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (tok < a.batch) {
                v = __ldcg(reinterpret_cast<const uint4*>(a.x + (int64_t)tok * xcols +
                                                          lg * per_group * kHeadDim) + c);
            }
            *reinterpret_cast<uint4*>(s_x + tok * x_pitch + c * 16) = v;
        }
    }
    __syncthreads();
    const uint32_t step = s_step;
    const uint32_t local_step = s_local_step;
    const int count = (SHARDED ? g.nranks : 1) * a.groups;  // KV heads of the whole model

    // ---- per-lane constants of the fragment loads ---------------------------------------
    const int r8 = lane & 7;
    // Weights (A operand): matrices ordered (rows 0-7, rows 8-15) x (k, k + 8).
    const uint32_t w_row_off = (((lane >> 3) & 1) * 8 + r8) * 128;
    const uint32_t w_xor = ((lane >> 4) ^ r8) << 4;
    // Activations (B operand): matrices ordered k, k + 8, k + 16, k + 24 of token r8.
    const uint32_t x_lane = smem_u32(s_x) + r8 * x_pitch + (lane >> 3) * 16;
    const int gid = lane >> 2;
    const int tig = lane & 3;

    int cons_stage = 0;
    uint32_t cons_parity = 0;
    bool timed_out = false;
    uint32_t task = 0;  // tasks this team has finished (selects the team's exchange buffer)
#pragma unroll 1
    for (int tile = worker; tile < tiles; tile += workers, ++task) {
        // One accumulator per block of 16 columns of a head (eight independent MMA chains, so
        // that the tensor pipe's latency is not paid per instruction); each runs over this
        // warp's heads of the KV head in ascending order. A warp whose wait ran out stops
        // reading but stays in step with its team (the barrier below has no time limit).
        float part[8][4];
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
            for (int i = 0; i < 4; ++i) part[ks][i] = 0.f;
        }
#pragma unroll 1
        for (int head = head0; head < head0 + team_heads; ++head) {
            const uint32_t tile_addr = ring + cons_stage * kHeadTileBytes + w_row_off;
            if (!timed_out && !wait_full(bars + cons_stage * 8, cons_parity)) timed_out = true;
            if (timed_out) continue;
            const uint32_t x_addr = x_lane + head * (kHeadDim * 2);
#pragma unroll
            for (int kp = 0; kp < 4; ++kp) {  // 32 columns per pass, ascending
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(x_addr + kp * 64, b0, b1, b2, b3);
                const uint32_t box = tile_addr + (kp >> 1) * kBoxBytes;
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(box + ((((kp & 1) * 4) << 4) ^ w_xor), a0, a1, a2, a3);
                mma_bf16_16816(part[2 * kp], a0, a1, a2, a3, b0, b1);
                ldmatrix_x4(box + ((((kp & 1) * 4 + 2) << 4) ^ w_xor), a0, a1, a2, a3);
                mma_bf16_16816(part[2 * kp + 1], a0, a1, a2, a3, b2, b3);
            }
            if (++cons_stage == a.stages) {
                cons_stage = 0;
                cons_parity ^= 1u;
            }
            __syncwarp();
            issue();  // the stage is free again
        }
        // The eight block sums, added in ascending order.
        float acc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[i] = part[0][i];
#pragma unroll
            for (int ks = 1; ks < 8; ++ks) acc[i] += part[ks][i];
        }
        if (team == 2) {
            // The warp of the upper heads hands its sums to the warp of the lower heads, which
            // adds them (lower + upper) and carries the task on. Two buffers taken in turn: the
            // upper warp cannot be two tasks ahead of a barrier the lower one has not passed.
            float* hand = s_team[unit][task & 1u] + lane * 4;
            if (member == 1) {
#pragma unroll
                for (int i = 0; i < 4; ++i) hand[i] = acc[i];
            }
            if (unit == 0) {
                asm volatile("bar.sync 1, 64;" ::: "memory");
            } else {
                asm volatile("bar.sync 2, 64;" ::: "memory");
            }
            if (member == 1) continue;
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] += hand[i];
        }
        // acc[0..1]: row gid, tokens 2 tig and 2 tig + 1; acc[2..3]: row gid + 8. With a single
        // KV head in the whole model that is the result; otherwise each sum becomes a tagged
        // word, here or (sharded) in every rank's window, for the second phase below.
        if (count == 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int b = 2 * tig + (i & 1);
                if (b >= a.batch) continue;
                const int n = tile * kTileRows + gid + (i >> 1) * 8;
                __nv_bfloat16* out = output_at(a, b, n);
                const float before = a.residual != nullptr ? __bfloat162float(*out) : 0.f;
                *out = __float2bfloat16(before + (0.f + acc[i]));
            }
            continue;
        }
        // Fragment order -> [token][row] through shared memory, then contiguous runs.
        float* stage = s_stage[warp];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            stage[(2 * tig + (i & 1)) * kTileRows + gid + (i >> 1) * 8] = acc[i];
        }
        __syncwarp();
        const int nwords = a.batch * kTileRows;
        const int64_t base = word_index(a, lg, 0, tile * kTileRows);
        if (!SHARDED) {
            for (int w = lane; w < nwords; w += 32) {
                push_word(a.words + base + w, local_step, __float_as_uint(stage[w]));
            }
        } else {
            for (int p = 0; p < g.nranks; ++p) {
                unsigned long long* dst =
                    window_slot(g.windows[p], step, g.nranks, g.rank, g.slot_bytes) + base;
                for (int w = lane; w < nwords; w += 32) {
                    push_word(dst + w, step, __float_as_uint(stage[w]));
                }
            }
        }
        __syncwarp();  // the next tile overwrites the staging row
    }

    // ---- second phase: every CTA finishes its share of the outputs -----------------------
    // All KV-head sums of the model, own ones included, are read back as words (those of other
    // CTAs and ranks may still be on their way: bounded polls), added in ascending order, and
    // the residual is updated. Nothing in the streaming loop above ever waits for another warp.
    if (count > 1) {
        const int64_t outputs = (int64_t)a.batch * a.hidden;
        for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < outputs && !timed_out;
             o += (int64_t)gridDim.x * blockDim.x) {
            const int ob = (int)(o / a.hidden), on = (int)(o % a.hidden);
            auto word_at = [&](int idx, uint32_t* tag) -> const unsigned long long* {
                const int r = idx / a.groups;
                const int64_t word = word_index(a, idx - r * a.groups, ob, on);
                if (SHARDED) {
                    *tag = step;
                    return window_slot(g.windows[g.rank], step, g.nranks, r, g.slot_bytes) + word;
                }
                *tag = local_step;
                return a.words + word;
            };
            __nv_bfloat16* out = output_at(a, ob, on);
            // The old value travels while the words are polled.
            const float before = a.residual != nullptr ? __bfloat162float(*out) : 0.f;
            float total = 0.f;
            const unsigned long long start = global_timer();
            for (int base = 0; base < count; base += 8) {
                // All loads of a batch of eight travel together; late words are asked for again.
                unsigned long long got[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint32_t tag;
                    if (base + i < count) got[i] = load_word(word_at(base + i, &tag));
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (base + i >= count) continue;
                    uint32_t tag;
                    const unsigned long long* src = word_at(base + i, &tag);
                    while ((uint32_t)(got[i] >> 32) != tag) {
                        if (global_timer() - start > kGatherWaitNs) {
                            timed_out = true;
                            break;
                        }
                        got[i] = load_word(src);
                    }
                    total += __uint_as_float((uint32_t)got[i]);
                }
            }
            if (!timed_out) *out = __float2bfloat16(before + total);
        }
    }
    if (timed_out) s_timed_out = 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_timed_out && a.status != nullptr) atomicExch(a.status, 2);
        // The last CTA to finish advances the launch counters for the next launch.
        if (a.ctrl != nullptr) {
            const uint32_t ticket = atomicAdd(&a.ctrl->ticket_out, 1u);
            if (ticket == gridDim.x - 1) {
                a.ctrl->ticket_out = 0;
                a.ctrl->step = s_local_step;
            }
        }
        if (SHARDED) {
            WindowCtrl* ctrl = window_ctrl(g.windows[g.rank], g.slot_bytes, g.nranks);
            if (s_timed_out) ctrl->status = 1;
            const uint32_t ticket = atomicAdd(&ctrl->ticket_out, 1u);
            if (ticket == gridDim.x - 1) {
                ctrl->ticket_out = 0;
                ctrl->step = s_step;
            }
        }
    }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr size_t kCtrlBytes = 256;

size_t workspace_bytes(int hidden, int groups) {
    if (groups <= 1) return 0;
    return kCtrlBytes + (size_t)groups * kProjTokens * hidden * sizeof(unsigned long long);
}

// Destinations of the split form (packed QKV projection); null for the residual form.
struct SplitOut {
    void* q;
    void* k;
    void* v;
    int32_t q_rows;
    int32_t kv_rows;
};

int validate(const gqa_oproj_params* p, const SplitOut* split) {
    if (p == nullptr) return GQA_ERR_NULL;
    if (p->attn_out == nullptr || p->weight == nullptr) return GQA_ERR_NULL;
    if (split == nullptr ? p->residual == nullptr
                         : (split->q == nullptr || split->k == nullptr || split->v == nullptr)) {
        return GQA_ERR_NULL;
    }
    if (p->head_dim != kHeadDim || p->batch <= 0 || p->hidden <= 0 || p->hidden % kTileRows != 0) {
        return GQA_ERR_SHAPE;
    }
    const int heads = p->num_q_heads;
    if (heads <= 0 || p->num_kv_heads <= 0 || heads % p->num_kv_heads != 0 ||
        heads / p->num_kv_heads > kMaxHeadsPerGroup) {
        return GQA_ERR_SHAPE;
    }
    if (p->weight_ld < (int64_t)heads * kHeadDim || p->weight_ld % 8 != 0) return GQA_ERR_SHAPE;
    if (!aligned16(p->attn_out) || !aligned16(p->weight)) return GQA_ERR_ALIGN;
    const size_t need = workspace_bytes(p->hidden, p->num_kv_heads);
    if (need != 0) {
        if (p->workspace == nullptr) return GQA_ERR_NULL;
        if (p->workspace_bytes < need) return GQA_ERR_WORKSPACE;
        if (!aligned16(p->workspace)) return GQA_ERR_ALIGN;
    }
    return GQA_OK;
}

size_t smem_bytes(int warps, int stages, int per_group) {
    return 1024 + (size_t)warps * stages * kHeadTileBytes +
           (size_t)kProjTokens * (per_group * kHeadDim * 2 + 16) + (size_t)warps * stages * 8;
}

// Ring depth per warp and CTAs per SM; "GQA_OPROJ_SHAPE=stages,ctas" overrides (tuning).
void oproj_shape(int* stages, int* ctas_per_sm) {
    *stages = 3;
    *ctas_per_sm = 3;
    static const char* env = std::getenv("GQA_OPROJ_SHAPE");
    int s = 0, c = 0;
    if (env != nullptr && std::sscanf(env, "%d,%d", &s, &c) == 2 && s >= 1 && s <= 12 && c >= 1 &&
        c <= 4) {
        *stages = s;
        *ctas_per_sm = c;
    }
}

int run(const gqa_oproj_params* p, const SplitOut* split, gqa_comm* comm) {
    const int rc = validate(p, split);
    if (rc != GQA_OK) return rc;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(p->stream);
    int32_t sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        return GQA_ERR_CUDA;
    }
    const int groups = p->num_kv_heads;
    const int per_group = p->num_q_heads / groups;
    const int tiles = p->hidden / kTileRows;
    int stages = 0, ctas_per_sm = 0;
    oproj_shape(&stages, &ctas_per_sm);
    // The shared-memory limit is a per-device property of the kernels: raise it once per device.
    {
        static std::mutex mu;
        static bool raised[64] = {};
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64) return GQA_ERR_CUDA;
        if (!raised[dev]) {
            if (cudaFuncSetAttribute(oproj_residual_kernel<false>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kMaxSmem) != cudaSuccess ||
                cudaFuncSetAttribute(oproj_residual_kernel<true>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kMaxSmem) != cudaSuccess) {
                return GQA_ERR_CUDA;
            }
            raised[dev] = true;
        }
    }
    // Every CTA of the grid waits, in its finishing phase, for words written by the others:
    // the whole grid must be resident at once. Wide groups need more shared memory per CTA,
    // so fewer CTAs fit an SM than the tuned number: ask the runtime.
    {
        const size_t full = smem_bytes(kProjMaxWarps, stages, per_group);
        if (full > (size_t)kMaxSmem) return GQA_ERR_SHAPE;
        int fit = 0;
        const cudaError_t oe =
            comm != nullptr && gqa_comm_nranks(comm) > 1
                ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&fit, oproj_residual_kernel<true>,
                                                                kProjMaxWarps * 32, full)
                : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&fit, oproj_residual_kernel<false>,
                                                                kProjMaxWarps * 32, full);
        if (oe != cudaSuccess || fit < 1) return GQA_ERR_CUDA;
        if (ctas_per_sm > fit) ctas_per_sm = fit;
    }
    // A task (16-row tile, KV head) belongs to a team: one warp, or - when the KV head has an
    // even number of query heads - two warps of a CTA that each stream half of them and add
    // their sums. With single warps the Qwen3-32B projection has 2560 tasks for 1776 warp
    // slots: 1280 warps take two each and a third of the slots stay empty, so the SMs that got
    // three CTAs stream half as much again as those that got two and the launch ends with
    // them. Teams of two make it 888 slots of three tasks each.
    static const bool teams_off = [] {
        const char* v = std::getenv("GQA_OPROJ_TEAM");
        return v != nullptr && v[0] == '1';
    }();
    const int team = (!teams_off && per_group >= 2 && per_group % 2 == 0) ? 2 : 1;
    const int units_max = kProjMaxWarps / team;  // teams per CTA
    // Every team gets the same number of tiles (k) of its KV head, or one fewer: as many
    // teams as the GPU holds at once, but no more than tiles; small problems use narrower
    // CTAs so that they still reach every SM.
    int ctas_per_group = ctas_per_sm * sms / groups;
    if (ctas_per_group < 1) ctas_per_group = 1;
    const int k = (tiles + ctas_per_group * units_max - 1) / (ctas_per_group * units_max);
    const int workers = (tiles + k - 1) / k;  // teams per KV head
    int warps = kProjMaxWarps;
    if ((int64_t)workers * groups * team < (int64_t)sms * kProjMaxWarps) {
        warps = (int)((int64_t)workers * groups * team / sms) / team * team;
        if (warps < team) warps = team;
    }
    const int units = warps / team;
    const int grid = (workers + units - 1) / units * groups;
    const size_t smem = smem_bytes(warps, stages, per_group);
    if (smem > (size_t)kMaxSmem) return GQA_ERR_SHAPE;
    CUtensorMap wmap;
    const int mrc = cached_matrix_map(p->weight, (int64_t)p->num_q_heads * kHeadDim, p->hidden,
                                      p->weight_ld, &wmap);
    if (mrc != GQA_OK) return mrc;
    // More than 8 tokens: one pass over the weights per 8 (each its own exchange step).
    for (int b0 = 0; b0 < p->batch; b0 += kProjTokens) {
        OprojArgs a;
        std::memset(&a, 0, sizeof(a));
        a.batch = p->batch - b0 < kProjTokens ? p->batch - b0 : kProjTokens;
        a.x = static_cast<const __nv_bfloat16*>(p->attn_out) +
              (int64_t)b0 * p->num_q_heads * kHeadDim;
        if (split == nullptr) {
            a.residual = static_cast<__nv_bfloat16*>(p->residual) + (int64_t)b0 * p->hidden;
        } else {
            a.q_rows = split->q_rows;
            a.kv_rows = split->kv_rows;
            a.q_out = static_cast<__nv_bfloat16*>(split->q) + (int64_t)b0 * split->q_rows;
            a.k_out = static_cast<__nv_bfloat16*>(split->k) + (int64_t)b0 * split->kv_rows;
            a.v_out = static_cast<__nv_bfloat16*>(split->v) + (int64_t)b0 * split->kv_rows;
        }
        if (groups > 1) {
            a.ctrl = static_cast<WindowCtrl*>(p->workspace);
            a.words = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(p->workspace) +
                                                            kCtrlBytes);
        }
        a.status = p->status_dev;
        a.hidden = p->hidden;
        a.heads = p->num_q_heads;
        a.groups = groups;
        a.stages = stages;
        a.team = team;
        PeerGatherArgs g;
        std::memset(&g, 0, sizeof(g));
        cudaError_t e;
        if (comm != nullptr && gqa_comm_nranks(comm) > 1) {
            const size_t bytes = (size_t)groups * a.batch * p->hidden * sizeof(float);
            const int crc = comm_peer_args(comm, bytes, p->status_dev, &g);
            if (crc != GQA_OK) return crc;
            e = launch_pdl(oproj_residual_kernel<true>, dim3(grid), dim3(32 * warps), smem, stream,
                           wmap, a, g);
        } else {
            e = launch_pdl(oproj_residual_kernel<false>, dim3(grid), dim3(32 * warps), smem,
                           stream, wmap, a, g);
        }
        if (e != cudaSuccess) return GQA_ERR_CUDA;
    }
    return GQA_OK;
}

}  // namespace
}  // namespace gqa

extern "C" {

size_t gqa_oproj_workspace_bytes(int32_t hidden, int32_t num_kv_heads) {
    if (hidden <= 0 || num_kv_heads <= 0) return 0;
    return gqa::workspace_bytes(hidden, num_kv_heads);
}

int gqa_oproj_residual(const gqa_oproj_params* p) { return gqa::run(p, nullptr, nullptr); }

int gqa_oproj_residual_sharded(const gqa_oproj_params* p, gqa_comm* comm) {
    if (comm == nullptr) return GQA_ERR_NULL;
    return gqa::run(p, nullptr, comm);
}

// The packed QKV projection runs on the same kernel: its input columns are cut into "heads"
// of 128 and groups of up to 8 heads, which only fixes the summation order.
static int qkv_groups(int32_t hidden) {
    const int heads = hidden / gqa::kHeadDim;
    int per_group = 8;
    while (heads % per_group != 0) --per_group;
    return heads / per_group;
}

size_t gqa_qkv_workspace_bytes(int32_t hidden, int32_t num_q_heads, int32_t num_kv_heads) {
    if (hidden <= 0 || hidden % gqa::kHeadDim != 0 || num_q_heads <= 0 || num_kv_heads <= 0) {
        return 0;
    }
    return gqa::workspace_bytes((num_q_heads + 2 * num_kv_heads) * gqa::kHeadDim,
                                qkv_groups(hidden));
}

int gqa_qkv_gemv(const gqa_qkv_params* p) {
    if (p == nullptr) return GQA_ERR_NULL;
    if (p->hidden <= 0 || p->hidden % gqa::kHeadDim != 0 || p->head_dim != gqa::kHeadDim ||
        p->num_q_heads <= 0 || p->num_kv_heads <= 0) {
        return GQA_ERR_SHAPE;
    }
    gqa_oproj_params o;
    std::memset(&o, 0, sizeof(o));
    o.batch = p->batch;
    o.hidden = (p->num_q_heads + 2 * p->num_kv_heads) * gqa::kHeadDim;  // output rows
    o.num_q_heads = p->hidden / gqa::kHeadDim;                          // input column heads
    o.num_kv_heads = qkv_groups(p->hidden);
    o.head_dim = gqa::kHeadDim;
    o.weight_ld = p->weight_ld;
    o.attn_out = p->x;
    o.weight = p->weight;
    o.workspace = p->workspace;
    o.workspace_bytes = p->workspace_bytes;
    o.status_dev = p->status_dev;
    o.stream = p->stream;
    const gqa::SplitOut split = {p->q_out, p->k_out, p->v_out, p->num_q_heads * gqa::kHeadDim,
                                 p->num_kv_heads * gqa::kHeadDim};
    return gqa::run(&o, &split, nullptr);
}

}  // extern "C"
