// BF16 streaming decode-attention kernel for sm_100a.
//
// Takes the place of the reference's flashattention_gqa_cp_async_kernel and
// flashdecoding_gqa_split_kernel (code/source/op/kernel/cuda/mha_kernel.cu:44-208, :210-388),
// which launch one CTA per QUERY head (so K/V are fetched `kv_mul` times) and cut the context
// every 32 keys. Here a CTA owns work items of one KV head: K and V leave HBM once and serve
// the whole query group.
//
// Data path. Every warp runs its own ring of STAGES stages. A stage holds KEYS consecutive
// keys: K [2][KEYS][64] and V [2][KEYS][64] BF16 (the 128 channels split in two 128-byte
// halves so that the 128-byte swizzle applies), KEYS * 512 bytes, filled by four 4-D bulk
// tensor copies whose completion is counted on the stage's mbarrier. Lane 0 of the warp refills a stage as soon
// as the warp has finished reading it, so each warp keeps STAGES chunks in flight and the
// CTA keeps WARPS * STAGES * 16 KiB in flight, with no CTA-wide synchronisation inside an
// item.
//
// Math. Scores are computed transposed, S^T[key][column] = K[key][:] . Q[column][:], on tensor
// cores (mma.sync m16n8k16, BF16 in, FP32 out) with the 16 keys on M and the columns of the
// unit on N. A column is a (query token, query head) pair: a decode step has one token and
// the (up to 8) heads of the group fill one N tile; with several query tokens per sequence
// (the reference prefills token by token through its decode kernel, main/main_qwen3.cpp:58-65)
// the tokens sit side by side on N, NT tiles of 8 columns, and column (t, n) sees keys
// 0 .. len - q_tokens + t only (a causal limit per column). Online softmax runs in FP32 in
// the exp2 domain; probabilities are rounded to BF16 (the row sum uses the rounded values, so
// the weights still sum to one), transposed with movmatrix and used as the B operand of
// O^T[channel][column] += V^T[channel][key] . P^T.
//
// Each warp keeps (m, l, O) for the chunks it consumed; at the end of an item the warps are
// merged through shared memory in warp order and the CTA writes either the final BF16
// output (unit not split) or an FP32 partial record for the combine kernel.
//
// FUSED adds the stage the reference runs in front of attention
// (fused_qk_norm_rope_kernel, code/source/op/kernel/cuda/rmsnorm_kernel.cu:205-290, and the
// KV-row placement of code/source/model/model.cpp:90-107) to the same launch: every CTA
// normalises and rotates the raw query rows of its unit itself (front_math.cuh: the same
// operations, hence the same bits, as the stand-alone front kernel), and the warp that
// consumes the stage holding a new token's position computes that token's key row, copies its
// value row, patches both into the staged tile in shared memory and appends them to the cache
// in HBM. Nothing else in the launch reads those cache rows, so no ordering between CTAs is
// needed.
//
// CLUSTER launches one thread-block cluster per unit with one CTA per split (at most 16): each
// CTA streams its split, leaves its (O, m, l) in its own shared memory, and after a cluster
// barrier the CTAs of the cluster merge the splits by reading one another's shared memory
// (distributed shared memory) and write the final rows. Short contexts, where the whole launch
// is one wave of CTAs and a second launch costs as much as the streaming, then need no combine
// kernel and no trip through the scratch. The merge performs the combine kernel's operations in
// the combine kernel's order, so both paths give the same bits.
#include <mutex>

#include "decode_kernels.cuh"
#include "front_math.cuh"
#include "ptx.cuh"
#include "work_map.cuh"

namespace gqa {

namespace {

constexpr int kOPitch = 132;                        // floats per column in the merge buffer
constexpr int kQPitch = 136;                        // BF16 per column of the rotated-query buffer
constexpr uint64_t kWaitBudgetNs = 2000000000ull;   // bounded wait for a staged chunk

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits for a stage to fill. Returns false when the budget ran out. The clock is read only
// now and then: reading it goes through the same queue as the loads and stores.
__device__ __forceinline__ bool wait_stage(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t start = 0;
    for (uint32_t tries = 1;; ++tries) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((tries & 255u) == 0) {
            const uint64_t now = global_timer_ns();
            if (start == 0) start = now;
            if (now - start > kWaitBudgetNs) return false;
        }
    }
}

struct Cursor {
    int32_t next;   // position of the item after the current one
    int32_t k;
    int32_t k_end;
    int32_t k_new;  // first stage that holds a position of the new tokens
    int32_t b;
    int32_t hk;
    bool valid;
};

}  // namespace

template <int WARPS, int STAGES, int KEYS, int OCC, int NT, bool FUSED, bool CLUSTER>
__global__ void __launch_bounds__(WARPS * 32, OCC)
gqa_decode_stream_bf16(const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const DecodeArgs a,
                       const FusedFrontArgs ff) {
    constexpr int kHalfBytes = KEYS * 128;       // one 64-channel half of K or V of a stage
    constexpr int kTileBytes = 2 * kHalfBytes;   // K or V of a stage
    constexpr int kStageBytes = 2 * kTileBytes;  // K + V
    constexpr int MT = KEYS / 16;                // 16-key MMA tiles per stage
    constexpr int kCols = 8 * NT;                // columns of the MMA N side
    extern __shared__ uint8_t smem_raw[];
    // The swizzle pattern is a function of the shared-memory address: stages sit on 1 KiB.
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* ring_all = smem;
    float* s_o = reinterpret_cast<float*>(ring_all + WARPS * STAGES * kStageBytes);
    float* s_m = s_o + WARPS * kCols * kOPitch;
    float* s_l = s_m + WARPS * kCols;
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_l + WARPS * kCols);
    __nv_bfloat16* s_q = reinterpret_cast<__nv_bfloat16*>(s_bar + WARPS * STAGES);
    float* s_rec = reinterpret_cast<float*>(s_q + (FUSED ? kCols * kQPitch : 0));
    int32_t* s_tables = reinterpret_cast<int32_t*>(s_rec + (CLUSTER ? kCols * (kHeadDim + 2) : 0));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < WARPS * STAGES; ++i) mbar_init(smem_u32(&s_bar[i]), 1);
        mbar_init_fence();
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
    }
    // The next kernel of the stream may be scheduled from now on (it waits for this one's
    // results itself before it reads them).
    pdl_launch_dependents();
    // Everything up to pdl_wait() overlaps the previous kernel of the stream. With
    // a.early_prefetch the caller has promised that nothing still running ahead of this
    // kernel writes cache rows other than the new positions of each sequence, nor the
    // lengths or the block table: stages that do not hold a new position are then
    // requested before the wait, which hides the DRAM ramp behind the predecessor's tail.
    // (FUSED: this kernel writes the new rows itself, so every stage may be requested.)
    if (!a.early_prefetch) pdl_wait();
    const WorkTables tables = build_work_tables(a, s_tables);
    __syncthreads();

    // The CTA's work is a walk over positions [pos_begin, pos_end). Persistent grid: items
    // blockIdx.x, blockIdx.x + gridDim.x, ... Even cut: this CTA's share of the flat sequence
    // of cells, one piece per unit it touches. Cluster launch: the one item this CTA's place
    // in its cluster stands for (or none).
    Item own = {};
    const bool has_own = CLUSTER ? cluster_item(a, tables, &own) : false;
    const bool even = !CLUSTER && a.even_ctas > 0;
    int32_t pos_begin = 0, pos_end = has_own ? 1 : 0;
    if (!CLUSTER) {
        const int32_t total = total_items(a, tables);
        const int32_t ctas = even_ctas(a, total);
        pos_begin = even ? even_begin(blockIdx.x, total, ctas) : (int32_t)blockIdx.x;
        pos_end = even ? even_begin(blockIdx.x + 1, total, ctas) : total;
    }
    // The item at a position, the index of its partial record and the position after it.
    auto fetch = [&](int32_t pos) -> Step {
        if (CLUSTER) return Step{own, 0, pos_end, true};
        if (even) return even_piece(a, tables, pos, pos_end, blockIdx.x);
        return Step{decode_item(a, tables, pos), pos, pos + (int32_t)gridDim.x, true};
    };
    const int32_t group = a.group;
    const int32_t q_tokens = a.q_tokens;
    const int32_t cols = group * q_tokens;
    const uint64_t policy = l2_policy_evict_first();
    const uint32_t ring = smem_u32(ring_all + warp * STAGES * kStageBytes);
    const uint32_t bars = smem_u32(&s_bar[warp * STAGES]);

    // ---- producer side: this warp's stage sequence across the CTA's items ----------------
    Cursor prod;
    prod.next = pos_begin;
    prod.k = 0;
    prod.k_end = 0;
    prod.k_new = 0;
    prod.b = 0;
    prod.hk = 0;
    prod.valid = true;
    auto normalize = [&](Cursor& c) {
        while (c.valid && c.k >= c.k_end) {
            if (c.next >= pos_end) {
                c.valid = false;
            } else {
                const Step st = fetch(c.next);
                const Item& it = st.it;
                c.next = st.next;
                if (!st.valid) {
                    c.valid = false;
                    break;
                }
                c.b = it.b;
                c.hk = it.hk;
                c.k = it.chunk_begin * kChunkKeys / KEYS + warp;
                c.k_end = ceil_div(min(it.len, it.chunk_end * kChunkKeys), KEYS);
                c.k_new = (it.len - q_tokens) / KEYS;
            }
        }
    };
    normalize(prod);
    uint32_t produced = 0;
    auto issue = [&]() {
        if (!prod.valid) return;
        const uint32_t stage = produced % STAGES;
        const int32_t t0 = prod.k * KEYS;
        int32_t blk = a.fixed_block;
        int32_t tok = t0;
        if (a.block_table != nullptr) {
            const int32_t lb = t0 / a.block_tokens;
            tok = t0 - lb * a.block_tokens;
            blk = __ldg(a.block_table + (int64_t)prod.b * a.blocks_per_seq + lb);
        }
        if (lane == 0) {
            // A block id outside the cache reads as zeros (the copy engine fills what lies
            // outside the tensor) and is reported.
            if ((uint32_t)blk >= (uint32_t)a.num_blocks) raise_status(a, kStatusBadInput);
            const uint32_t bar = bars + stage * 8;
            const uint32_t dst = ring + stage * kStageBytes;
            fence_proxy_async();
            mbar_arrive_expect_tx(bar, kStageBytes);
            // The tensor maps list their dimensions by ascending stride: (channel, head,
            // token, block) for the reference cache, (channel, token, head, block) for the pool.
            const int32_t c1 = a.head_before_token ? prod.hk : tok;
            const int32_t c2 = a.head_before_token ? tok : prod.hk;
            tma_load_4d(dst, &tmap_k, bar, 0, c1, c2, blk, policy);
            tma_load_4d(dst + kHalfBytes, &tmap_k, bar, 64, c1, c2, blk, policy);
            tma_load_4d(dst + kTileBytes, &tmap_v, bar, 0, c1, c2, blk, policy);
            tma_load_4d(dst + kTileBytes + kHalfBytes, &tmap_v, bar, 64, c1, c2, blk, policy);
        }
        ++produced;
        prod.k += WARPS;
        normalize(prod);
    };
    if (a.early_prefetch) {
#pragma unroll 1
        for (int s = 0; s < STAGES; ++s) {
            if (!prod.valid || (!FUSED && prod.k >= prod.k_new)) break;
            issue();
        }
        pdl_wait();
    }
#pragma unroll 1
    for (int s = (int)produced; s < STAGES; ++s) issue();

    // ---- per-lane constants of the fragment loads ----------------------------------------
    const int r8 = lane & 7;
    // K (A operand of S^T, not transposed): matrices ordered (keys 0-7, keys 8-15) x (d, d+8).
    const uint32_t k_row_off = (((lane >> 3) & 1) * 8 + r8) * 128;
    const uint32_t k_xor = ((lane >> 4) ^ r8) << 4;
    // V (A operand of O^T, transposed on load): matrices ordered (d, d+8) x (keys 0-7, 8-15).
    const uint32_t v_row_off = ((lane >> 4) * 8 + r8) * 128;
    const uint32_t v_xor = (((lane >> 3) & 1) ^ r8) << 4;

    uint32_t consumed = 0;
    bool dead = false;

#pragma unroll 1
    for (int32_t pos = pos_begin, pos_next = 0; pos < pos_end; pos = pos_next) {
        const Step step = fetch(pos);
        if (!step.valid) break;
        const Item& it = step.it;
        const int32_t record = step.record;
        pos_next = step.next;
        const int32_t new_lo = it.len - q_tokens;  // position of the first query token

        // Row of column c in q / out: [sequence][token][query head][channel].
        auto q_row_of = [&](int c) -> int64_t {
            const int t = c / group;
            const int n = c - t * group;
            return (((int64_t)it.b * a.q_token_stride + a.q_token_first + t) * a.num_q_heads +
                    (int64_t)it.hk * group + n) * kHeadDim;
        };

        if (FUSED) {
            // QK-Norm + RoPE of this unit's raw query rows, one warp per column.
            const __nv_bfloat16* wei = reinterpret_cast<const __nv_bfloat16*>(ff.qk_weight);
            for (int c = warp; c < cols; c += WARPS) {
                const int32_t pos = new_lo + c / group;
                const bool tab = ff.sin_cache != nullptr && pos < ff.table_len;
                const float* sin_row = tab ? ff.sin_cache + (int64_t)pos * (kHeadDim / 2) : nullptr;
                const float* cos_row = tab ? ff.cos_cache + (int64_t)pos * (kHeadDim / 2) : nullptr;
                const int64_t row = q_row_of(c);
                __nv_bfloat16 y[4];
                front_norm_rope(reinterpret_cast<const __nv_bfloat16*>(a.q) + row, wei, sin_row,
                                cos_row, pos, ff.eps, lane, y);
#pragma unroll
                for (int i = 0; i < 4; ++i) s_q[c * kQPitch + lane + 32 * i] = y[i];
                if (it.split == 0 && ff.q_out != nullptr) {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(ff.q_out) + row;
#pragma unroll
                    for (int i = 0; i < 4; ++i) dst[lane + 32 * i] = y[i];
                }
            }
            __syncthreads();
        }

        // Query columns as B fragments: B[k = channel][n = column] = Q[column][channel].
        uint32_t qf[NT][8][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int c = nt * 8 + (lane >> 2);
            const __nv_bfloat16* qrow =
                FUSED ? s_q + c * kQPitch + 2 * (lane & 3)
                      : reinterpret_cast<const __nv_bfloat16*>(a.q) + q_row_of(c < cols ? c : 0) +
                            2 * (lane & 3);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                if (c < cols) {
                    if (FUSED) {
                        qf[nt][ks][0] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16);
                        qf[nt][ks][1] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8);
                    } else {
                        qf[nt][ks][0] = __ldcg(reinterpret_cast<const uint32_t*>(qrow + ks * 16));
                        qf[nt][ks][1] = __ldcg(reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8));
                    }
                } else {
                    qf[nt][ks][0] = 0u;
                    qf[nt][ks][1] = 0u;
                }
            }
        }

        const int32_t key_end = min(it.len, it.chunk_end * kChunkKeys);
        // Causal limit of this lane's columns (2 per N tile): keys [0, lim) are visible.
        int32_t lim[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = nt * 8 + 2 * (lane & 3) + e;
                const int t = c < cols ? c / group : q_tokens - 1;
                lim[nt][e] = min(key_end, new_lo + t + 1);
            }
        }
        const int32_t lim_min = min(key_end, new_lo + 1);

        float m[NT][2], l[NT][2];  // running maxima and this lane's share of the running sums
        float o[NT][8][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            m[nt][0] = -INFINITY; m[nt][1] = -INFINITY;
            l[nt][0] = 0.0f; l[nt][1] = 0.0f;
#pragma unroll
            for (int dt = 0; dt < 8; ++dt) {
                o[nt][dt][0] = 0.0f; o[nt][dt][1] = 0.0f; o[nt][dt][2] = 0.0f; o[nt][dt][3] = 0.0f;
            }
        }

        const int32_t k_end = ceil_div(key_end, KEYS);
#pragma unroll 1
        for (int32_t k = it.chunk_begin * kChunkKeys / KEYS + warp; k < k_end; k += WARPS) {
            if (dead) break;
            const uint32_t stage = consumed % STAGES;
            const uint32_t parity = (consumed / STAGES) & 1u;
            if (!wait_stage(bars + stage * 8, parity)) {
                dead = true;
                if (lane == 0) raise_status(a, kStatusStageTimeout);
                break;
            }
            const uint32_t kbase = ring + stage * kStageBytes;
            const uint32_t vbase = kbase + kTileBytes;
            const int32_t valid = key_end - k * KEYS;  // keys of this stage inside the item

            if (FUSED && (k + 1) * KEYS > new_lo) {
                // The stage holds positions of the new tokens, whose rows are not in the cache
                // yet: compute them, patch the staged tile and append them to the cache.
                uint8_t* kptr = ring_all + (warp * STAGES + stage) * kStageBytes;
                const __nv_bfloat16* wei =
                    reinterpret_cast<const __nv_bfloat16*>(ff.qk_weight) + kHeadDim;
#pragma unroll 1
                for (int t = 0; t < q_tokens; ++t) {
                    const int32_t pos = new_lo + t;
                    const int32_t r = pos - k * KEYS;
                    if (r < 0 || r >= KEYS) continue;
                    int32_t blk = a.fixed_block;
                    int32_t tok = pos;
                    if (a.block_table != nullptr) {
                        const int32_t lb = pos / a.block_tokens;
                        tok = pos - lb * a.block_tokens;
                        blk = __ldg(a.block_table + (int64_t)it.b * a.blocks_per_seq + lb);
                    }
                    const bool blk_ok = (uint32_t)blk < (uint32_t)a.num_blocks;
                    const int64_t cache_off = (int64_t)blk * a.stride_block +
                                              (int64_t)tok * a.stride_token +
                                              (int64_t)it.hk * a.stride_head;
                    const int64_t new_off =
                        (((int64_t)it.b * a.q_token_stride + a.q_token_first + t) * a.num_kv_heads +
                         it.hk) * kHeadDim;
                    const bool tab = ff.sin_cache != nullptr && pos < ff.table_len;
                    const float* sin_row = tab ? ff.sin_cache + (int64_t)pos * (kHeadDim / 2) : nullptr;
                    const float* cos_row = tab ? ff.cos_cache + (int64_t)pos * (kHeadDim / 2) : nullptr;
                    __nv_bfloat16 y[4];
                    front_norm_rope(reinterpret_cast<const __nv_bfloat16*>(ff.k_new) + new_off, wei,
                                    sin_row, cos_row, pos, ff.eps, lane, y);
                    __nv_bfloat16* k_dst = reinterpret_cast<__nv_bfloat16*>(
                                               const_cast<void*>(a.k_cache)) + cache_off;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int c64 = lane + 32 * (i & 1);
                        *reinterpret_cast<__nv_bfloat16*>(
                            kptr + (i >> 1) * kHalfBytes + r * 128 +
                            ((((c64 >> 3) ^ (r & 7))) << 4) + (c64 & 7) * 2) = y[i];
                        if (blk_ok) k_dst[lane + 32 * i] = y[i];
                    }
                    const uint2 vv = __ldcg(reinterpret_cast<const uint2*>(
                                                reinterpret_cast<const __nv_bfloat16*>(ff.v_new) +
                                                new_off) + lane);
                    *reinterpret_cast<uint2*>(kptr + kTileBytes + (lane >> 4) * kHalfBytes + r * 128 +
                                              (((((lane & 15) >> 1) ^ (r & 7))) << 4) +
                                              (lane & 1) * 8) = vv;
                    if (blk_ok) {
                        reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(
                            const_cast<void*>(a.v_cache)) + cache_off)[lane] = vv;
                    }
                }
                fence_proxy_async();  // these writes precede the next bulk copy into the stage
                __syncwarp();
            }

            if (valid < KEYS) {
                // Rows past the sequence end hold whatever the cache holds there. Zero those
                // V rows: their probabilities are zero, but 0 * NaN would still poison O.
                uint8_t* vptr = ring_all + (warp * STAGES + stage) * kStageBytes + kTileBytes;
                for (int idx = lane; idx < 2 * KEYS * 8; idx += 32) {
                    const int half = idx / (KEYS * 8);
                    const int row = (idx / 8) % KEYS;
                    if (row >= valid) {
                        *reinterpret_cast<uint4*>(vptr + half * kHalfBytes + row * 128 +
                                                  (idx & 7) * 16) = make_uint4(0, 0, 0, 0);
                    }
                }
                fence_proxy_async();  // these writes precede the next bulk copy into the stage
                __syncwarp();
            }

            // ---- S^T = K . Q^T for MT tiles of 16 keys ----------------------------------
            float s[NT][MT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    s[nt][mt][0] = 0.0f; s[nt][mt][1] = 0.0f; s[nt][mt][2] = 0.0f; s[nt][mt][3] = 0.0f;
                }
            }
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t col = ((uint32_t)((ks & 3) * 2) << 4) ^ k_xor;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint32_t a0, a1, a2, a3;
                    ldmatrix_x4(kbase + (ks >> 2) * kHalfBytes + mt * 2048 + k_row_off + col,
                                a0, a1, a2, a3);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        mma_bf16_16816(s[nt][mt], a0, a1, a2, a3, qf[nt][ks][0], qf[nt][ks][1]);
                    }
                }
            }

            // ---- online softmax (exp2 domain) -------------------------------------------
            uint32_t pb[NT][MT][2];
            bool rescale = false;
            float alpha[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) s[nt][mt][c] *= a.scale_log2;
                }
                if ((k + 1) * KEYS > lim_min) {
                    // Keys past the item's end and keys a column's token may not see yet.
                    const int32_t v0 = lim[nt][0] - k * KEYS;
                    const int32_t v1 = lim[nt][1] - k * KEYS;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const int key = mt * 16 + (lane >> 2);
                        if (key >= v0) s[nt][mt][0] = -INFINITY;
                        if (key >= v1) s[nt][mt][1] = -INFINITY;
                        if (key + 8 >= v0) s[nt][mt][2] = -INFINITY;
                        if (key + 8 >= v1) s[nt][mt][3] = -INFINITY;
                    }
                }
                float c0 = fmaxf(s[nt][0][0], s[nt][0][2]);
                float c1 = fmaxf(s[nt][0][1], s[nt][0][3]);
#pragma unroll
                for (int mt = 1; mt < MT; ++mt) {
                    c0 = fmaxf(c0, fmaxf(s[nt][mt][0], s[nt][mt][2]));
                    c1 = fmaxf(c1, fmaxf(s[nt][mt][1], s[nt][mt][3]));
                }
#pragma unroll
                for (int d = 4; d < 32; d <<= 1) {
                    c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, d));
                    c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, d));
                }
                const float n0 = fmaxf(m[nt][0], c0);
                const float n1 = fmaxf(m[nt][1], c1);
                const float e0 = safe_max(n0);
                const float e1 = safe_max(n1);
                alpha[nt][0] = ex2_approx(m[nt][0] - e0);
                alpha[nt][1] = ex2_approx(m[nt][1] - e1);
                m[nt][0] = n0;
                m[nt][1] = n1;

                float add0 = 0.0f, add1 = 0.0f;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint32_t p01 = pack_bf16(ex2_approx(s[nt][mt][0] - e0),
                                                   ex2_approx(s[nt][mt][1] - e1));
                    const uint32_t p23 = pack_bf16(ex2_approx(s[nt][mt][2] - e0),
                                                   ex2_approx(s[nt][mt][3] - e1));
                    add0 += bf16_lo_to_f32(p01) + bf16_lo_to_f32(p23);
                    add1 += bf16_hi_to_f32(p01) + bf16_hi_to_f32(p23);
                    pb[nt][mt][0] = movmatrix_trans(p01);
                    pb[nt][mt][1] = movmatrix_trans(p23);
                }
                l[nt][0] = l[nt][0] * alpha[nt][0] + add0;
                l[nt][1] = l[nt][1] * alpha[nt][1] + add1;
                rescale = rescale || (alpha[nt][0] != 1.0f) || (alpha[nt][1] != 1.0f);
            }
            if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int dt = 0; dt < 8; ++dt) {
                        o[nt][dt][0] *= alpha[nt][0]; o[nt][dt][1] *= alpha[nt][1];
                        o[nt][dt][2] *= alpha[nt][0]; o[nt][dt][3] *= alpha[nt][1];
                    }
                }
            }

            // ---- O^T += V^T . P^T ---------------------------------------------------------
#pragma unroll
            for (int dt = 0; dt < 8; ++dt) {
                const uint32_t col = ((uint32_t)((dt & 3) * 2) << 4) ^ v_xor;
#pragma unroll
                for (int kt = 0; kt < MT; ++kt) {
                    uint32_t a0, a1, a2, a3;
                    ldmatrix_x4_trans(vbase + (dt >> 2) * kHalfBytes + kt * 2048 + v_row_off + col,
                                      a0, a1, a2, a3);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        mma_bf16_16816(o[nt][dt], a0, a1, a2, a3, pb[nt][kt][0], pb[nt][kt][1]);
                    }
                }
            }

            ++consumed;
            __syncwarp();
            issue();  // refill the stage just read
        }

        // ---- merge the warps of this CTA ---------------------------------------------------
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int d = 4; d < 32; d <<= 1) {
                l[nt][0] += __shfl_xor_sync(0xffffffffu, l[nt][0], d);
                l[nt][1] += __shfl_xor_sync(0xffffffffu, l[nt][1], d);
            }
            const int c0 = nt * 8 + 2 * (lane & 3);
            if (lane < 4) {
                s_m[warp * kCols + c0] = m[nt][0];
                s_m[warp * kCols + c0 + 1] = m[nt][1];
                s_l[warp * kCols + c0] = l[nt][0];
                s_l[warp * kCols + c0 + 1] = l[nt][1];
            }
            float* dst = s_o + (warp * kCols + c0) * kOPitch + (lane >> 2);
#pragma unroll
            for (int dt = 0; dt < 8; ++dt) {
                dst[dt * 16] = o[nt][dt][0];
                dst[kOPitch + dt * 16] = o[nt][dt][1];
                dst[dt * 16 + 8] = o[nt][dt][2];
                dst[kOPitch + dt * 16 + 8] = o[nt][dt][3];
            }
        }
        __syncthreads();
        {
            const bool final_out = (it.nsplits == 1) && a.always_partial == 0;
            // A record that does not fit the scratch is not written (lengths read from the
            // device may have outgrown what the scratch was sized for).
            const bool fits = CLUSTER || final_out || record < a.item_capacity;
            if (!fits && threadIdx.x == 0) raise_status(a, kStatusBadInput);
            float* rec = CLUSTER ? s_rec : a.workspace + (int64_t)record * cols * (kHeadDim + 2);
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out);
            for (int idx = threadIdx.x; fits && idx < cols * kHeadDim; idx += WARPS * 32) {
                const int n = idx >> 7;
                const int d = idx & (kHeadDim - 1);
                float mx = s_m[n];
#pragma unroll
                for (int w = 1; w < WARPS; ++w) mx = fmaxf(mx, s_m[w * kCols + n]);
                const float ref = safe_max(mx);
                float acc = 0.0f, lsum = 0.0f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    const float f = ex2_approx(s_m[w * kCols + n] - ref);
                    acc += s_o[(w * kCols + n) * kOPitch + d] * f;
                    lsum += s_l[w * kCols + n] * f;
                }
                if (final_out) {
                    out[q_row_of(n) + d] = __float2bfloat16(acc / lsum);
                } else {
                    rec[idx] = acc;
                    if (d == 0) {
                        rec[cols * kHeadDim + n] = mx;
                        rec[cols * kHeadDim + cols + n] = lsum;
                    }
                }
            }
        }
        __syncthreads();
    }

    if (CLUSTER) {
        // Every CTA of the cluster gets here, with or without an item. After the barrier the
        // records of the unit's splits are readable in their CTAs' shared memory; the rows are
        // dealt to all threads of the cluster. The arithmetic is gqa_decode_combine's for a
        // unit of up to 8 splits: weights relative to the largest maximum, products rounded
        // before they are added, splits in ascending order.
        cluster_sync_all();
        const int32_t csize = a.cluster_size;
        if (own.nsplits > 1) {
            const int32_t rank = own.split;
            const uint32_t rec_base = smem_u32(s_rec);
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out);
            for (int idx = rank * (WARPS * 32) + threadIdx.x; idx < cols * kHeadDim;
                 idx += csize * (WARPS * 32)) {
                const int n = idx >> 7;
                const int d = idx & (kHeadDim - 1);
                constexpr int kMaxSplits = 16;
                float ms[kMaxSplits], ls[kMaxSplits], os[kMaxSplits];
#pragma unroll
                for (int sp = 0; sp < kMaxSplits; ++sp) {
                    if (sp < own.nsplits) {
                        const uint32_t base = cluster_map(rec_base, (uint32_t)sp);
                        ms[sp] = ld_cluster_f32(base + (cols * kHeadDim + n) * 4);
                        ls[sp] = ld_cluster_f32(base + (cols * kHeadDim + cols + n) * 4);
                        os[sp] = ld_cluster_f32(base + idx * 4);
                    } else {
                        ms[sp] = -INFINITY; ls[sp] = 0.0f; os[sp] = 0.0f;
                    }
                }
                float tmax = ms[0];
#pragma unroll
                for (int sp = 1; sp < kMaxSplits; ++sp) tmax = fmaxf(tmax, ms[sp]);
                const float ref = safe_max(tmax);
                float wgt[kMaxSplits];
                float ltile = 0.0f;
#pragma unroll
                for (int sp = 0; sp < kMaxSplits; ++sp) {
                    wgt[sp] = ex2_approx(ms[sp] - ref);
                    if (sp < own.nsplits) ltile = __fmaf_rn(ls[sp], wgt[sp], ltile);
                }
                // Eight slots (split s in slot s % 8, ascending inside a slot), slots added in
                // ascending order: the combine kernel's order for up to 32 splits.
                float acc = 0.0f;
#pragma unroll
                for (int slot = 0; slot < 8; ++slot) {
                    float part = 0.0f;
                    if (slot < own.nsplits) part = __fmaf_rn(os[slot], wgt[slot], part);
                    if (slot + 8 < own.nsplits) part = __fmaf_rn(os[slot + 8], wgt[slot + 8], part);
                    acc = slot == 0 ? part : __fadd_rn(acc, part);
                }
                const int t = n / group;
                const int64_t row = (((int64_t)own.b * a.q_token_stride + a.q_token_first + t) *
                                         a.num_q_heads + (int64_t)own.hk * group + (n - t * group)) *
                                    kHeadDim;
                out[row + d] = __float2bfloat16(acc / ltile);
            }
        }
        // No CTA may leave (and give up its shared memory) while another still reads it.
        cluster_sync_all();
    }
}

size_t stream_bf16_smem_bytes(int warps, int stages, int keys, int n_tiles, bool fused,
                              bool cluster, int batch_for_tables) {
    const size_t cols = 8 * (size_t)n_tiles;
    size_t bytes = 1024;  // alignment slack
    bytes += (size_t)warps * stages * keys * 512;
    bytes += (size_t)warps * cols * kOPitch * sizeof(float);
    bytes += 2 * (size_t)warps * cols * sizeof(float);
    bytes += (size_t)warps * stages * sizeof(uint64_t);
    if (fused) bytes += cols * kQPitch * sizeof(__nv_bfloat16);
    if (cluster) bytes += cols * (kHeadDim + 2) * sizeof(float);
    bytes += 2 * ((size_t)batch_for_tables + 1) * sizeof(int32_t);
    return bytes;
}

template <int WARPS, int STAGES, int KEYS, int OCC, int NT, bool FUSED, bool CLUSTER>
static cudaError_t launch_variant(const CUtensorMap& tk, const CUtensorMap& tv,
                                  const DecodeArgs& args, const FusedFrontArgs& ff, int grid,
                                  cudaStream_t stream, int* max_clusters) {
    const int tables = args.seq_lens_dev != nullptr ? args.batch : 0;
    const size_t smem = stream_bf16_smem_bytes(WARPS, STAGES, KEYS, NT, FUSED, CLUSTER, tables);
    auto kernel = gqa_decode_stream_bf16<WARPS, STAGES, KEYS, OCC, NT, FUSED, CLUSTER>;
    // The attribute is per function and per device.
    static std::mutex mu;
    static size_t configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || configured[dev] < smem) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) configured[dev] = smem;
        }
    }
    if (CLUSTER && args.cluster_size > 8) {
        // Clusters of more than 8 CTAs are not portable across GPUs: ask for them explicitly.
        static bool allowed[64] = {};
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !allowed[dev]) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) allowed[dev] = true;
        }
    }
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    if (CLUSTER) {
        attrs[1].id = cudaLaunchAttributeClusterDimension;
        attrs[1].val.clusterDim.x = (unsigned)args.cluster_size;
        attrs[1].val.clusterDim.y = 1;
        attrs[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
        if (max_clusters != nullptr) {
            // Query only: how many clusters of this size the GPU holds at once.
            *max_clusters = 0;
            return cudaOccupancyMaxActiveClusters(max_clusters, kernel, &cfg);
        }
    }
    return cudaLaunchKernelEx(&cfg, kernel, tk, tv, args, ff);
}

template <bool CLUSTER>
static cudaError_t launch_by_shape(const CUtensorMap& tk, const CUtensorMap& tv,
                                   const DecodeArgs& args, const FusedFrontArgs* fused, int grid,
                                   cudaStream_t stream, int* max_clusters) {
    constexpr StreamShape S = kDefaultStreamShape;
    FusedFrontArgs ff = {};
    if (fused != nullptr) ff = *fused;
    const int cols = args.group * args.q_tokens;
    if (cols <= 8) {
        return fused != nullptr
                   ? launch_variant<S.warps, S.stages, S.keys, 1, 1, true, CLUSTER>(
                         tk, tv, args, ff, grid, stream, max_clusters)
                   : launch_variant<S.warps, S.stages, S.keys, 1, 1, false, CLUSTER>(
                         tk, tv, args, ff, grid, stream, max_clusters);
    }
    if (cols <= 16) {
        return fused != nullptr
                   ? launch_variant<S.warps, S.stages, S.keys, 1, 2, true, CLUSTER>(
                         tk, tv, args, ff, grid, stream, max_clusters)
                   : launch_variant<S.warps, S.stages, S.keys, 1, 2, false, CLUSTER>(
                         tk, tv, args, ff, grid, stream, max_clusters);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_stream_bf16(const CUtensorMap& tk, const CUtensorMap& tv, const DecodeArgs& args,
                               const FusedFrontArgs* fused, int grid, cudaStream_t stream) {
    return args.cluster_size > 0
               ? launch_by_shape<true>(tk, tv, args, fused, grid, stream, nullptr)
               : launch_by_shape<false>(tk, tv, args, fused, grid, stream, nullptr);
}

int stream_bf16_max_clusters(const CUtensorMap& tk, const CUtensorMap& tv, const DecodeArgs& args,
                             const FusedFrontArgs* fused, int grid) {
    int clusters = 0;
    if (args.cluster_size <= 0 ||
        launch_by_shape<true>(tk, tv, args, fused, grid, nullptr, &clusters) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return clusters;
}

}  // namespace gqa
