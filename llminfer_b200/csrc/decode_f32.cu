// FP32 decode attention (FP32 q / cache / output) and the LSE combine kernel.
//
// The FP32 kernel covers what the reference's CPU backend computes in FP32
// (code/source/op/kernel/cpu/mha_kernel.cpp:34-110) and its op tests compare at 1e-5
// (test/test_op/test_op_mha.cpp:62): scores, softmax and the weighted sum all stay in FP32 on
// CUDA cores, with accurate exp2f. It uses the same item decomposition and partial-record
// format as the BF16 kernel, so one combine kernel serves both. It is a parity path for
// short FP32 caches, not a bandwidth path.
//
// The combine kernel takes the place of flashdecoding_gqa_combine_kernel
// (code/source/op/kernel/cuda/mha_kernel.cu:399-438): out = sum_s O_s 2^(m_s - M) /
// sum_s l_s 2^(m_s - M), splits added in a fixed order.
#include <cstring>

#include "decode_kernels.cuh"
#include "peer_window.cuh"
#include "ptx.cuh"
#include "work_map.cuh"

namespace gqa {

namespace {

constexpr int kF32Warps = 4;
constexpr int kF32Threads = kF32Warps * 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}

__device__ __forceinline__ const float* cache_row(const DecodeArgs& a, const void* base,
                                                  int32_t b, int32_t hk, int32_t t) {
    int32_t blk = a.fixed_block;
    int32_t tok = t;
    if (a.block_table != nullptr) {
        const int32_t lb = t / a.block_tokens;
        tok = t - lb * a.block_tokens;
        blk = __ldg(a.block_table + (int64_t)b * a.blocks_per_seq + lb);
        // A block id outside the cache is reported and read as block 0: no wild address.
        if ((uint32_t)blk >= (uint32_t)a.num_blocks) {
            if ((threadIdx.x & 31) == 0) raise_status(a, kStatusBadInput);
            blk = 0;
        }
    }
    return reinterpret_cast<const float*>(base) + (int64_t)blk * a.stride_block +
           (int64_t)tok * a.stride_token + (int64_t)hk * a.stride_head;
}

}  // namespace

// G: query heads per kv head handled per pass (group <= G).
template <int G>
__global__ void __launch_bounds__(kF32Threads) gqa_decode_stream_f32(const DecodeArgs a) {
    __shared__ float s_o[kF32Warps][G][kHeadDim];
    __shared__ float s_m[kF32Warps][G];
    __shared__ float s_l[kF32Warps][G];
    extern __shared__ int32_t s_tables[];

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    const WorkTables tables = build_work_tables(a, s_tables);
    const int32_t n_items = total_items(a, tables);
    const int32_t group = a.group;

    for (int32_t item = blockIdx.x; item < n_items; item += gridDim.x) {
        const Item it = decode_item(a, tables, item);

        float4 q[G];
        float m[G], l[G];
        float4 o[G];
#pragma unroll
        for (int n = 0; n < G; ++n) {
            q[n] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (n < group) {
                q[n] = __ldcg(reinterpret_cast<const float4*>(
                                 reinterpret_cast<const float*>(a.q) +
                                 ((int64_t)it.b * a.num_q_heads + (int64_t)it.hk * group + n) *
                                     kHeadDim) + lane);
            }
            m[n] = -INFINITY;
            l[n] = 0.f;
            o[n] = make_float4(0.f, 0.f, 0.f, 0.f);
        }

        for (int32_t k = it.chunk_begin + warp; k < it.chunk_end; k += kF32Warps) {
            const int32_t t0 = k * kChunkKeys;
            const int32_t valid = min(kChunkKeys, it.len - t0);

            // The 32 rows of a chunk lie in one cache block, stride_token apart.
            const float4* krow = reinterpret_cast<const float4*>(
                                     cache_row(a, a.k_cache, it.b, it.hk, t0)) + lane;
            const float4* vrow = reinterpret_cast<const float4*>(
                                     cache_row(a, a.v_cache, it.b, it.hk, t0)) + lane;
            const int64_t row_f4 = a.stride_token / 4;

            // Scores: lane j ends up holding the G scores of key t0 + j. Rows are fetched
            // eight at a time so that their latencies overlap.
            float sc[G];
#pragma unroll
            for (int n = 0; n < G; ++n) sc[n] = -INFINITY;
#pragma unroll 1
            for (int32_t j0 = 0; j0 < valid; j0 += 8) {
                float4 kv[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    kv[jj] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (j0 + jj < valid) kv[jj] = __ldg(krow + (int64_t)(j0 + jj) * row_f4);
                }
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
#pragma unroll
                    for (int n = 0; n < G; ++n) {
                        float part = q[n].x * kv[jj].x + q[n].y * kv[jj].y + q[n].z * kv[jj].z +
                                     q[n].w * kv[jj].w;
                        part = warp_sum(part);
                        if (lane == j0 + jj) sc[n] = part * a.scale_log2;
                    }
                }
            }

            float p[G];
#pragma unroll
            for (int n = 0; n < G; ++n) {
                const float cmax = warp_max(sc[n]);
                const float mnew = fmaxf(m[n], cmax);
                const float alpha = exp2f(m[n] - mnew);
                p[n] = (lane < valid) ? exp2f(sc[n] - mnew) : 0.f;
                l[n] = l[n] * alpha + p[n];
                o[n].x *= alpha; o[n].y *= alpha; o[n].z *= alpha; o[n].w *= alpha;
                m[n] = mnew;
            }

#pragma unroll 1
            for (int32_t j0 = 0; j0 < valid; j0 += 8) {
                float4 vv[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    vv[jj] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (j0 + jj < valid) vv[jj] = __ldg(vrow + (int64_t)(j0 + jj) * row_f4);
                }
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
#pragma unroll
                    for (int n = 0; n < G; ++n) {
                        // Keys past the end have p = 0 and a zero row.
                        const float pj = __shfl_sync(0xffffffffu, p[n], (j0 + jj) & 31);
                        o[n].x += pj * vv[jj].x; o[n].y += pj * vv[jj].y;
                        o[n].z += pj * vv[jj].z; o[n].w += pj * vv[jj].w;
                    }
                }
            }
        }

#pragma unroll
        for (int n = 0; n < G; ++n) {
            const float lt = warp_sum(l[n]);
            if (lane == 0) {
                s_m[warp][n] = m[n];
                s_l[warp][n] = lt;
            }
            reinterpret_cast<float4*>(&s_o[warp][n][0])[lane] = o[n];
        }
        __syncthreads();
        {
            const bool final_out = (it.nsplits == 1) && a.always_partial == 0;
            const bool fits = final_out || item < a.item_capacity;
            if (!fits && threadIdx.x == 0) raise_status(a, kStatusBadInput);
            float* rec = a.workspace + (int64_t)item * group * (kHeadDim + 2);
            float* out = reinterpret_cast<float*>(a.out) +
                ((int64_t)it.b * a.num_q_heads + (int64_t)it.hk * group) * kHeadDim;
            for (int idx = threadIdx.x; fits && idx < group * kHeadDim; idx += kF32Threads) {
                const int n = idx >> 7;
                const int d = idx & (kHeadDim - 1);
                float mx = s_m[0][n];
#pragma unroll
                for (int w = 1; w < kF32Warps; ++w) mx = fmaxf(mx, s_m[w][n]);
                const float ref = safe_max(mx);
                float acc = 0.f, lsum = 0.f;
#pragma unroll
                for (int w = 0; w < kF32Warps; ++w) {
                    const float f = exp2f(s_m[w][n] - ref);
                    acc += s_o[w][n][d] * f;
                    lsum += s_l[w][n] * f;
                }
                if (final_out) {
                    out[idx] = acc / lsum;
                } else {
                    rec[idx] = acc;
                    if (d == 0) {
                        rec[group * kHeadDim + n] = mx;
                        rec[group * kHeadDim + group + n] = lsum;
                    }
                }
            }
        }
        __syncthreads();
    }
}

constexpr int kCombineLocal = 0;   // merge the splits of a unit
constexpr int kCombineGather = 1;  // ... and exchange the finished rows (KV-head-parallel)
constexpr int kCombineSeqPar = 2;  // ... and merge with the other ranks' slices of the keys
constexpr int kCombineRecord = 3;  // ... and leave the row's record instead of the output
constexpr int kCombineWideGrid = 160;  // largest grid that runs with 4 lanes per channel
constexpr int kCombineTile = 64;   // splits merged per pass
constexpr int kCombineSlots = 8;   // partial sums per channel per pass, whatever the CTA width
constexpr int kRecWords = kHeadDim + 2;  // a row's record: 128 channel sums, maximum, row sum

// Merges the records of `count` slices of one row's keys (each: channel sum d relative to the
// slice's maximum, the maximum in the log2 domain, the row sum) in ascending order, so every
// caller that holds the same records gets the same bits. A slice without keys has the record
// (0, -inf, 0) and drops out. rec(r, w) returns word w of slice r.
template <bool FAST_EXP, typename Rec>
__device__ __forceinline__ float merge_slices(int count, int d, Rec rec) {
    float m_all = rec(0, kHeadDim);
    for (int r = 1; r < count; ++r) m_all = fmaxf(m_all, rec(r, kHeadDim));
    const float ref = safe_max(m_all);
    float l_all = 0.f, o_all = 0.f;
    for (int r = 0; r < count; ++r) {
        const float diff = rec(r, kHeadDim) - ref;
        const float w = FAST_EXP ? ex2_approx(diff) : exp2f(diff);
        l_all += rec(r, kHeadDim + 1) * w;
        o_all += rec(r, d) * w;
    }
    return o_all / l_all;
}

// One CTA per output row (sequence, query token, query head) with LANES threads per output
// channel. The splits of a
// pass are dealt to 8 slots (split s goes to slot s % 8); a thread owns 8 / LANES slots and
// adds each slot's splits in ascending order, then the slots are added in ascending order.
// The result therefore does not depend on LANES, which is only a matter of how many threads
// share the loads: 4 lanes (512 threads, few enough registers to sit on an SM next to a CTA of
// the streaming kernel, so that neither kernel delays the other's early launch) for small
// grids, 2 for grids that would not fit the GPU in one wave at that size. Every load of a pass (O rows, m and l) is issued before any
// is used, so a pass costs one trip to L2; longer split lists fold pass by pass with a running
// (M, L). Partial records are read with L1-bypassing loads: the kernel that wrote them may
// still have been running when this one started.
//
// GATHER adds the exchange between the GPUs of a KV-head-parallel node to the same kernel:
// each CTA pushes its finished row, as step-tagged 8-byte words, into its place in every
// rank's peer window with plain stores over NVLink, then polls (with a time limit) the same
// row of every rank in its own window and writes them to the gathered output. A row leaves as
// soon as it is merged, so the transfer of the first rows overlaps the merge of the others and
// the separate gather launch goes away. Units that were not split are pushed from the output
// the streaming kernel wrote. Used only when every CTA of the grid is resident at once.
template <bool BF16_OUT, int LANES, int MODE>
__global__ void __launch_bounds__(kHeadDim * LANES)
    gqa_decode_combine(const DecodeArgs a, const PeerGatherArgs g) {
    constexpr int kOwn = kCombineSlots / LANES;            // slots per thread
    constexpr int kPerSlot = kCombineTile / kCombineSlots;  // splits per slot per pass
    extern __shared__ int32_t s_tables[];
    __shared__ float s_m[kCombineTile];
    __shared__ float s_l[kCombineTile];
    __shared__ float s_part[kCombineSlots][kHeadDim];
    pdl_launch_dependents();
    // The streaming kernel ahead of this one does not write the lengths. When the caller has
    // promised that nothing else still running does either (early_prefetch), the work tables
    // are built, and the address translation of this row's records warmed, while that kernel
    // is still running: after the wait only the records themselves remain to be fetched.
    if (!a.early_prefetch) pdl_wait();
    const WorkTables tables = build_work_tables(a, s_tables);
    // blockIdx.x = (sequence * q_tokens + token) * num_q_heads + head.
    const int32_t bt = blockIdx.x / a.num_q_heads;
    const int32_t h = blockIdx.x - bt * a.num_q_heads;
    const int32_t b = bt / a.q_tokens;
    const int32_t group = a.group;
    const int32_t cols = group * a.q_tokens;
    const int32_t hk = h / group;
    const int32_t col = (bt - b * a.q_tokens) * group + (h - hk * group);
    int32_t first, nsplits;
    unit_items(a, tables, b, hk, &first, &nsplits);
    const bool records = MODE == kCombineSeqPar || MODE == kCombineRecord;
    if ((nsplits > 1 || (records && nsplits == 1)) && first + nsplits > a.item_capacity) {
        // The unit's records did not fit the scratch (the streaming kernel skipped them and
        // raised the status word): nothing to read.
        if (threadIdx.x == 0) raise_status(a, kStatusBadInput);
        nsplits = 0;
    }
    if (a.early_prefetch) {
        if (nsplits > 1 || (records && nsplits == 1)) {
            const int64_t rec_floats = (int64_t)cols * (kHeadDim + 2);
            for (int32_t s = threadIdx.x; s < nsplits; s += blockDim.x) {
                prefetch_l2(a.workspace + (int64_t)(first + s) * rec_floats + col * kHeadDim);
            }
        }
        pdl_wait();
    }
    // Not split: the streaming kernel already wrote the final output.
    if (MODE == kCombineLocal && nsplits <= 1) return;

    const int d = threadIdx.x & (kHeadDim - 1);
    const int j = threadIdx.x >> 7;
    // The row's place in out: [sequence][token of the whole run][query head][channel].
    const int64_t o_idx = (((int64_t)b * a.q_token_stride + a.q_token_first + (bt - b * a.q_tokens)) *
                               a.num_q_heads + h) * kHeadDim + d;
    float result = 0.f;  // the finished channel, held by the threads with j == 0
    float m_run = -INFINITY, l_run = 0.f, acc = 0.f;
    if (nsplits > 1 || records) {
        const int64_t rec_floats = (int64_t)cols * (kHeadDim + 2);
        const float* rec0 = a.workspace + (int64_t)first * rec_floats;
        const float* m_base = rec0 + cols * kHeadDim + col;
        const float* l_base = m_base + cols;
        const float* o_base = rec0 + col * kHeadDim + d;

        for (int32_t base = 0; base < nsplits; base += kCombineTile) {
            const int32_t cnt = min(kCombineTile, nsplits - base);
            float o[kOwn][kPerSlot];
            float ml[kOwn][kPerSlot];
#pragma unroll
            for (int t = 0; t < kOwn; ++t) {
#pragma unroll
                for (int r = 0; r < kPerSlot; ++r) {
                    const int32_t s = (j + t * LANES) + r * kCombineSlots;
                    o[t][r] = 0.f;
                    ml[t][r] = 0.f;
                    if (s < cnt) {
                        const int64_t off = (int64_t)(base + s) * rec_floats;
                        o[t][r] = __ldcg(o_base + off);
                        if (d == 0) ml[t][r] = __ldcg(m_base + off);
                        if (d == 1) ml[t][r] = __ldcg(l_base + off);
                    }
                }
            }
            if (d < 2) {
#pragma unroll
                for (int t = 0; t < kOwn; ++t) {
#pragma unroll
                    for (int r = 0; r < kPerSlot; ++r) {
                        const int32_t s = (j + t * LANES) + r * kCombineSlots;
                        if (s < cnt) (d == 0 ? s_m : s_l)[s] = ml[t][r];
                    }
                }
            }
            __syncthreads();
            float tmax = s_m[0];
            for (int32_t i = 1; i < cnt; ++i) tmax = fmaxf(tmax, s_m[i]);
            const float m_new = fmaxf(m_run, tmax);
            // A split whose keys are all hidden from this row's token has m = -inf, l = 0.
            const float ref = safe_max(m_new);
            const float rescale = BF16_OUT ? ex2_approx(m_run - ref) : exp2f(m_run - ref);
            float ltile = 0.f;
            for (int32_t i = 0; i < cnt; ++i) {
                const float w = BF16_OUT ? ex2_approx(s_m[i] - ref) : exp2f(s_m[i] - ref);
                ltile = __fmaf_rn(s_l[i], w, ltile);
            }
#pragma unroll
            for (int t = 0; t < kOwn; ++t) {
                float part = 0.f;
#pragma unroll
                for (int r = 0; r < kPerSlot; ++r) {
                    const int32_t s = (j + t * LANES) + r * kCombineSlots;
                    if (s < cnt) {
                        const float w = BF16_OUT ? ex2_approx(s_m[s] - ref) : exp2f(s_m[s] - ref);
                        part = __fmaf_rn(o[t][r], w, part);
                    }
                }
                s_part[j + t * LANES][d] = part;
            }
            __syncthreads();
            if (j == 0) {
                // Explicit roundings: the in-cluster merge of the streaming kernel performs the
                // same operations and must give the same bits.
                float tile_acc = s_part[0][d];
#pragma unroll
                for (int v = 1; v < kCombineSlots; ++v) tile_acc = __fadd_rn(tile_acc, s_part[v][d]);
                acc = __fmaf_rn(acc, rescale, tile_acc);
            }
            l_run = __fmaf_rn(l_run, rescale, ltile);
            m_run = m_new;
            __syncthreads();  // the next pass overwrites s_m, s_l and s_part
        }
        if (j == 0 && !records) {
            result = acc / l_run;
            if (BF16_OUT) {
                reinterpret_cast<__nv_bfloat16*>(a.out)[o_idx] = __float2bfloat16(result);
            } else {
                reinterpret_cast<float*>(a.out)[o_idx] = result;
            }
        }
    } else if (MODE == kCombineGather && j == 0) {
        result = BF16_OUT ? __bfloat162float(__ldcg(reinterpret_cast<const __nv_bfloat16*>(a.out) + o_idx))
                          : __ldcg(reinterpret_cast<const float*>(a.out) + o_idx);
    }
    if (MODE == kCombineLocal) return;
    if (MODE == kCombineRecord) {
        // The row's record goes to the caller, who merges it with other slices' records.
        float* dst = reinterpret_cast<float*>(g.recv) + (int64_t)blockIdx.x * kRecWords;
        if (j == 0) dst[d] = acc;
        if (threadIdx.x == 0) {
            dst[kHeadDim] = m_run;
            dst[kHeadDim + 1] = l_run;
        }
        return;
    }

    // ---- exchange with the other ranks ----
    __shared__ uint32_t s_step;
    __shared__ int s_timed_out;
    uint8_t* mine = g.windows[g.rank];
    WindowCtrl* ctrl = window_ctrl(mine, g.slot_bytes, g.nranks);
    if (threadIdx.x == 0) {
        s_step = *reinterpret_cast<volatile uint32_t*>(&ctrl->step) + 1;
        s_timed_out = 0;
    }
    bool timed_out = false;
    if (MODE == kCombineGather) {
        // The finished row goes to every rank and the same row of every rank comes back.
        constexpr int kRowWords = BF16_OUT ? kHeadDim / 2 : kHeadDim;
        __shared__ uint32_t s_row[kRowWords];
        if (j == 0) {
            if (BF16_OUT) {
                const uint32_t bits = __bfloat16_as_ushort(__float2bfloat16(result));
                const uint32_t next = __shfl_down_sync(0xffffffffu, bits, 1);
                if ((d & 1) == 0) s_row[d >> 1] = bits | (next << 16);
            } else {
                s_row[d] = __float_as_uint(result);
            }
        }
        __syncthreads();
        const uint32_t step = s_step;
        const uint64_t row_off = (uint64_t)blockIdx.x * kRowWords;
        const int total = kRowWords * g.nranks;
        for (int i = threadIdx.x; i < total; i += kHeadDim * LANES) {
            const int p = i / kRowWords;
            const int w = i - p * kRowWords;
            push_word(window_slot(g.windows[p], step, g.nranks, g.rank, g.slot_bytes) + row_off + w,
                      step, s_row[w]);
        }
        const unsigned long long start = global_timer();
        for (int i = threadIdx.x; i < total && !timed_out; i += kHeadDim * LANES) {
            const int p = i / kRowWords;
            const int w = i - p * kRowWords;
            uint32_t data;
            if (poll_word(window_slot(mine, step, g.nranks, p, g.slot_bytes) + row_off + w, step,
                          start, &data)) {
                g.recv[(uint64_t)p * g.words + row_off + w] = data;
            } else {
                timed_out = true;
            }
        }
    } else {
        // Sequence-parallel: this rank saw a slice of the row's keys. Its record goes to every
        // other rank; the records of all ranks are merged in rank order, so every rank gets the
        // same bits.
        __shared__ uint32_t s_rec[kMaxPeers][kRecWords];
        if (j == 0) s_rec[g.rank][d] = __float_as_uint(acc);
        if (threadIdx.x == 0) {
            s_rec[g.rank][kHeadDim] = __float_as_uint(m_run);
            s_rec[g.rank][kHeadDim + 1] = __float_as_uint(l_run);
        }
        __syncthreads();
        const uint32_t step = s_step;
        const uint64_t row_off = (uint64_t)blockIdx.x * kRecWords;
        const int total = kRecWords * g.nranks;
        for (int i = threadIdx.x; i < total; i += kHeadDim * LANES) {
            const int p = i / kRecWords;
            const int w = i - p * kRecWords;
            if (p == g.rank) continue;
            push_word(window_slot(g.windows[p], step, g.nranks, g.rank, g.slot_bytes) + row_off + w,
                      step, s_rec[g.rank][w]);
        }
        const unsigned long long start = global_timer();
        for (int i = threadIdx.x; i < total && !timed_out; i += kHeadDim * LANES) {
            const int p = i / kRecWords;
            const int w = i - p * kRecWords;
            if (p == g.rank) continue;
            uint32_t data;
            if (poll_word(window_slot(mine, step, g.nranks, p, g.slot_bytes) + row_off + w, step,
                          start, &data)) {
                s_rec[p][w] = data;
            } else {
                timed_out = true;
            }
        }
        if (timed_out) s_timed_out = 1;
        __syncthreads();
        if (j == 0 && s_timed_out == 0) {
            const float merged = merge_slices<BF16_OUT>(
                g.nranks, d, [&](int r, int w) { return __uint_as_float(s_rec[r][w]); });
            if (BF16_OUT) {
                reinterpret_cast<__nv_bfloat16*>(a.out)[o_idx] = __float2bfloat16(merged);
            } else {
                reinterpret_cast<float*>(a.out)[o_idx] = merged;
            }
        }
    }
    if (timed_out) s_timed_out = 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_timed_out) {
            ctrl->status = 1;
            if (g.status != nullptr) atomicExch(g.status, kStatusPeerTimeout);
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

// Stand-alone merge of slice records (what the sequence-parallel exchange does after the
// records have arrived): records [nparts][rows][130], one thread per output channel.
template <bool BF16_OUT>
__global__ void __launch_bounds__(kHeadDim)
    gqa_merge_partials_kernel(const float* __restrict__ records, int32_t nparts, int64_t rows,
                              void* out) {
    const int64_t row = blockIdx.x;
    const int d = threadIdx.x;
    const float merged = merge_slices<BF16_OUT>(nparts, d, [&](int r, int w) {
        return __ldg(records + ((int64_t)r * rows + row) * kRecWords + w);
    });
    if (BF16_OUT) {
        reinterpret_cast<__nv_bfloat16*>(out)[row * kHeadDim + d] = __float2bfloat16(merged);
    } else {
        reinterpret_cast<float*>(out)[row * kHeadDim + d] = merged;
    }
}

cudaError_t launch_merge_partials(const float* records, int32_t nparts, int64_t rows,
                                  bool bf16_out, void* out, cudaStream_t stream) {
    if (bf16_out) {
        gqa_merge_partials_kernel<true><<<(unsigned)rows, kHeadDim, 0, stream>>>(records, nparts,
                                                                                rows, out);
    } else {
        gqa_merge_partials_kernel<false><<<(unsigned)rows, kHeadDim, 0, stream>>>(records, nparts,
                                                                                 rows, out);
    }
    return cudaGetLastError();
}

cudaError_t launch_stream_f32(const DecodeArgs& args, int grid, cudaStream_t stream) {
    const size_t smem =
        args.seq_lens_dev != nullptr ? 2 * ((size_t)args.batch + 1) * sizeof(int32_t) : 0;
    if (args.group <= 2) {
        return launch_pdl(gqa_decode_stream_f32<2>, dim3(grid), dim3(kF32Threads), smem, stream, args);
    } else if (args.group <= 4) {
        return launch_pdl(gqa_decode_stream_f32<4>, dim3(grid), dim3(kF32Threads), smem, stream, args);
    }
    return launch_pdl(gqa_decode_stream_f32<8>, dim3(grid), dim3(kF32Threads), smem, stream, args);
}

cudaError_t launch_combine(const DecodeArgs& args, bool bf16_out, cudaStream_t stream,
                           const PeerGatherArgs* gather, CombineKind kind) {
    const size_t smem =
        args.seq_lens_dev != nullptr ? 2 * ((size_t)args.batch + 1) * sizeof(int32_t) : 0;
    const int grid = args.batch * args.q_tokens * args.num_q_heads;
    const bool wide = grid <= kCombineWideGrid;
    PeerGatherArgs g;
    std::memset(&g, 0, sizeof(g));
    if (gather != nullptr) g = *gather;
    const dim3 block(kHeadDim * (wide ? 4 : 2));
#define GQA_COMBINE(MODE)                                                                       \
    (bf16_out ? (wide ? launch_pdl(gqa_decode_combine<true, 4, MODE>, dim3(grid), block, smem,  \
                                   stream, args, g)                                             \
                      : launch_pdl(gqa_decode_combine<true, 2, MODE>, dim3(grid), block, smem,  \
                                   stream, args, g))                                            \
              : (wide ? launch_pdl(gqa_decode_combine<false, 4, MODE>, dim3(grid), block, smem, \
                                   stream, args, g)                                             \
                      : launch_pdl(gqa_decode_combine<false, 2, MODE>, dim3(grid), block, smem, \
                                   stream, args, g)))
    switch (kind) {
        case CombineKind::kSeqPar:
            if (gather == nullptr) return cudaErrorInvalidValue;
            return GQA_COMBINE(kCombineSeqPar);
        case CombineKind::kRecord:
            if (gather == nullptr) return cudaErrorInvalidValue;
            return GQA_COMBINE(kCombineRecord);
        case CombineKind::kGather:
            if (gather == nullptr || !wide) return cudaErrorInvalidValue;  // combine_can_gather()
            return GQA_COMBINE(kCombineGather);
        case CombineKind::kLocal:
            break;
    }
    return GQA_COMBINE(kCombineLocal);
#undef GQA_COMBINE
}

// CTAs of the combine kernel that one SM holds at once for a grid of this size (the exchange
// modes make every CTA wait for its peers, so the whole grid must be resident).
int combine_resident_ctas(int grid, int sm_count) {
    const bool wide = grid <= kCombineWideGrid;
    int per_sm = 0;
    const cudaError_t e =
        wide ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                   &per_sm, gqa_decode_combine<true, 4, kCombineSeqPar>, kHeadDim * 4, 0)
             : cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                   &per_sm, gqa_decode_combine<true, 2, kCombineSeqPar>, kHeadDim * 2, 0);
    if (e != cudaSuccess) return 0;
    return per_sm * sm_count;
}

bool combine_can_gather(int rows, int sm_count) {
    return rows <= kCombineWideGrid && rows <= sm_count;
}

}  // namespace gqa
