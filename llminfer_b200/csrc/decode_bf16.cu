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
// Math. Scores are computed transposed, S^T[key][head] = K[key][:] . Q[head][:], on tensor
// cores (mma.sync m16n8k16, BF16 in, FP32 out) with the 16 keys on M and the (up to 8) query
// heads of the group on N, so the group costs one MMA column block whatever its width.
// Online softmax runs in FP32 in the exp2 domain; probabilities are rounded to BF16 (the
// row sum uses the rounded values, so the weights still sum to one), transposed with
// movmatrix and used as the B operand of O^T[channel][head] += V^T[channel][key] . P^T.
//
// Each warp keeps (m, l, O) for the chunks it consumed; at the end of an item the warps are
// merged through shared memory in warp order and the CTA writes either the final BF16
// output (unit not split) or an FP32 partial record for the combine kernel.
#include "decode_kernels.cuh"
#include "ptx.cuh"
#include "work_map.cuh"

namespace gqa {

namespace {

constexpr int kOPitch = 132;                        // floats per head in the merge buffer
constexpr int kHeadsPad = 8;                        // MMA N
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
    int32_t item;
    int32_t k;
    int32_t k_end;
    int32_t k_last;  // stage holding the newest position of the sequence
    int32_t b;
    int32_t hk;
    bool valid;
};

}  // namespace

template <int WARPS, int STAGES, int KEYS, int OCC>
__global__ void __launch_bounds__(WARPS * 32, OCC)
gqa_decode_stream_bf16(const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const DecodeArgs a) {
    constexpr int kHalfBytes = KEYS * 128;       // one 64-channel half of K or V of a stage
    constexpr int kTileBytes = 2 * kHalfBytes;   // K or V of a stage
    constexpr int kStageBytes = 2 * kTileBytes;  // K + V
    constexpr int MT = KEYS / 16;                // 16-key MMA tiles per stage
    extern __shared__ uint8_t smem_raw[];
    // The swizzle pattern is a function of the shared-memory address: stages sit on 1 KiB.
    uint8_t* smem = reinterpret_cast<uint8_t*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* ring_all = smem;
    float* s_o = reinterpret_cast<float*>(ring_all + WARPS * STAGES * kStageBytes);
    float* s_m = s_o + WARPS * kHeadsPad * kOPitch;
    float* s_l = s_m + WARPS * kHeadsPad;
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_l + WARPS * kHeadsPad);
    int32_t* s_tables = reinterpret_cast<int32_t*>(s_bar + WARPS * STAGES);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    timeline_mark(0, a.fixed_block);

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
    // kernel writes cache rows other than the newest position of each sequence, nor the
    // lengths or the block table: stages that do not hold a newest position are then
    // requested before the wait, which hides the DRAM ramp behind the predecessor's tail.
    if (!a.early_prefetch) pdl_wait();
    timeline_mark(1, a.fixed_block);
    const WorkTables tables = build_work_tables(a, s_tables);
    __syncthreads();

    const int32_t n_items = total_items(a, tables);
    const int32_t group = a.group;
    const uint64_t policy = l2_policy_evict_first();
    const uint32_t ring = smem_u32(ring_all + warp * STAGES * kStageBytes);
    const uint32_t bars = smem_u32(&s_bar[warp * STAGES]);

    // ---- producer side: this warp's stage sequence across the CTA's items ----------------
    Cursor prod;
    prod.item = blockIdx.x - gridDim.x;
    prod.k = 0;
    prod.k_end = 0;
    prod.k_last = 0;
    prod.b = 0;
    prod.hk = 0;
    prod.valid = true;
    auto normalize = [&](Cursor& c) {
        while (c.valid && c.k >= c.k_end) {
            c.item += gridDim.x;
            if (c.item >= n_items) {
                c.valid = false;
            } else {
                const Item it = decode_item(a, tables, c.item);
                c.b = it.b;
                c.hk = it.hk;
                c.k = it.chunk_begin * kChunkKeys / KEYS + warp;
                c.k_end = ceil_div(min(it.len, it.chunk_end * kChunkKeys), KEYS);
                c.k_last = (it.len - 1) / KEYS;
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
            if (!prod.valid || prod.k == prod.k_last) break;
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
    for (int32_t item = blockIdx.x; item < n_items; item += gridDim.x) {
        const Item it = decode_item(a, tables, item);

        // Query group as B fragments: B[k = channel][n = head] = Q[head][channel].
        uint32_t qf[8][2];
        {
            const int n = lane >> 2;
            const __nv_bfloat16* qrow = reinterpret_cast<const __nv_bfloat16*>(a.q) +
                ((int64_t)it.b * a.num_q_heads + (int64_t)it.hk * group + n) * kHeadDim +
                2 * (lane & 3);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                if (n < group) {
                    qf[ks][0] = __ldcg(reinterpret_cast<const uint32_t*>(qrow + ks * 16));
                    qf[ks][1] = __ldcg(reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8));
                } else {
                    qf[ks][0] = 0u;
                    qf[ks][1] = 0u;
                }
            }
        }

        float m0 = -INFINITY, m1 = -INFINITY;  // running maxima of heads 2*(lane&3), +1
        float l0 = 0.0f, l1 = 0.0f;            // this lane's share of the running sums
        float o[8][4];
#pragma unroll
        for (int dt = 0; dt < 8; ++dt) {
            o[dt][0] = 0.0f; o[dt][1] = 0.0f; o[dt][2] = 0.0f; o[dt][3] = 0.0f;
        }

        const int32_t key_end = min(it.len, it.chunk_end * kChunkKeys);
        const int32_t k_end = ceil_div(key_end, KEYS);
#pragma unroll 1
        for (int32_t k = it.chunk_begin * kChunkKeys / KEYS + warp; k < k_end; k += WARPS) {
            if (dead) break;
            const uint32_t stage = consumed % STAGES;
            const uint32_t parity = (consumed / STAGES) & 1u;
            if (!wait_stage(bars + stage * 8, parity)) {
                dead = true;
                if (lane == 0 && a.status != nullptr) atomicExch(a.status, 1);
                break;
            }
            if (consumed == 0) {
                timeline_mark(2, a.fixed_block);
                timeline_cta(0);
                timeline_cta(1);
            }
            const uint32_t kbase = ring + stage * kStageBytes;
            const uint32_t vbase = kbase + kTileBytes;
            const int32_t valid = key_end - k * KEYS;  // keys of this stage inside the item

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
            float s[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                s[mt][0] = 0.0f; s[mt][1] = 0.0f; s[mt][2] = 0.0f; s[mt][3] = 0.0f;
            }
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint32_t col = ((uint32_t)((ks & 3) * 2) << 4) ^ k_xor;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint32_t a0, a1, a2, a3;
                    ldmatrix_x4(kbase + (ks >> 2) * kHalfBytes + mt * 2048 + k_row_off + col,
                                a0, a1, a2, a3);
                    mma_bf16_16816(s[mt], a0, a1, a2, a3, qf[ks][0], qf[ks][1]);
                }
            }

            // ---- online softmax (exp2 domain) -------------------------------------------
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int c = 0; c < 4; ++c) s[mt][c] *= a.scale_log2;
            }
            if (valid < KEYS) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int key = mt * 16 + (lane >> 2);
                    if (key >= valid) { s[mt][0] = -INFINITY; s[mt][1] = -INFINITY; }
                    if (key + 8 >= valid) { s[mt][2] = -INFINITY; s[mt][3] = -INFINITY; }
                }
            }
            float c0 = fmaxf(s[0][0], s[0][2]);
            float c1 = fmaxf(s[0][1], s[0][3]);
#pragma unroll
            for (int mt = 1; mt < MT; ++mt) {
                c0 = fmaxf(c0, fmaxf(s[mt][0], s[mt][2]));
                c1 = fmaxf(c1, fmaxf(s[mt][1], s[mt][3]));
            }
#pragma unroll
            for (int d = 4; d < 32; d <<= 1) {
                c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, d));
                c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, d));
            }
            const float n0 = fmaxf(m0, c0);
            const float n1 = fmaxf(m1, c1);
            const float alpha0 = ex2_approx(m0 - n0);
            const float alpha1 = ex2_approx(m1 - n1);
            m0 = n0;
            m1 = n1;

            uint32_t pb[MT][2];
            float add0 = 0.0f, add1 = 0.0f;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const uint32_t p01 = pack_bf16(ex2_approx(s[mt][0] - n0), ex2_approx(s[mt][1] - n1));
                const uint32_t p23 = pack_bf16(ex2_approx(s[mt][2] - n0), ex2_approx(s[mt][3] - n1));
                add0 += bf16_lo_to_f32(p01) + bf16_lo_to_f32(p23);
                add1 += bf16_hi_to_f32(p01) + bf16_hi_to_f32(p23);
                pb[mt][0] = movmatrix_trans(p01);
                pb[mt][1] = movmatrix_trans(p23);
            }
            l0 = l0 * alpha0 + add0;
            l1 = l1 * alpha1 + add1;
            if (__any_sync(0xffffffffu, (alpha0 != 1.0f) || (alpha1 != 1.0f))) {
#pragma unroll
                for (int dt = 0; dt < 8; ++dt) {
                    o[dt][0] *= alpha0; o[dt][1] *= alpha1;
                    o[dt][2] *= alpha0; o[dt][3] *= alpha1;
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
                    mma_bf16_16816(o[dt], a0, a1, a2, a3, pb[kt][0], pb[kt][1]);
                }
            }

            ++consumed;
            __syncwarp();
            issue();  // refill the stage just read
        }

        // ---- merge the warps of this CTA ---------------------------------------------------
        timeline_mark(3, a.fixed_block);
        timeline_cta(2);
#pragma unroll
        for (int d = 4; d < 32; d <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, d);
            l1 += __shfl_xor_sync(0xffffffffu, l1, d);
        }
        {
            const int h0 = 2 * (lane & 3);
            if (lane < 4) {
                s_m[warp * kHeadsPad + h0] = m0;
                s_m[warp * kHeadsPad + h0 + 1] = m1;
                s_l[warp * kHeadsPad + h0] = l0;
                s_l[warp * kHeadsPad + h0 + 1] = l1;
            }
            float* dst = s_o + (warp * kHeadsPad + h0) * kOPitch + (lane >> 2);
#pragma unroll
            for (int dt = 0; dt < 8; ++dt) {
                dst[dt * 16] = o[dt][0];
                dst[kOPitch + dt * 16] = o[dt][1];
                dst[dt * 16 + 8] = o[dt][2];
                dst[kOPitch + dt * 16 + 8] = o[dt][3];
            }
        }
        __syncthreads();
        {
            const bool final_out = (it.nsplits == 1) && a.always_partial == 0;
            float* rec = a.workspace + (int64_t)item * group * (kHeadDim + 2);
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out) +
                ((int64_t)it.b * a.num_q_heads + (int64_t)it.hk * group) * kHeadDim;
            for (int idx = threadIdx.x; idx < group * kHeadDim; idx += WARPS * 32) {
                const int n = idx >> 7;
                const int d = idx & (kHeadDim - 1);
                float mx = s_m[n];
#pragma unroll
                for (int w = 1; w < WARPS; ++w) mx = fmaxf(mx, s_m[w * kHeadsPad + n]);
                float acc = 0.0f, lsum = 0.0f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) {
                    const float f = ex2_approx(s_m[w * kHeadsPad + n] - mx);
                    acc += s_o[(w * kHeadsPad + n) * kOPitch + d] * f;
                    lsum += s_l[w * kHeadsPad + n] * f;
                }
                if (final_out) {
                    out[idx] = __float2bfloat16(acc / lsum);
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
    timeline_mark(4, a.fixed_block);
    timeline_cta(3);
}

#ifdef GQA_TIMELINE
__device__ unsigned long long g_timeline[64];
__device__ unsigned long long g_cta_marks[4 * 1024];
extern "C" int gqa_timeline_ctas(unsigned long long* host) {
    return cudaMemcpyFromSymbol(host, g_cta_marks, sizeof(unsigned long long) * 4096) ==
                   cudaSuccess ? 0 : -1;
}
extern "C" int gqa_timeline_read(unsigned long long* host64, int reset) {
    if (cudaMemcpyFromSymbol(host64, g_timeline, sizeof(unsigned long long) * 64) != cudaSuccess) {
        return -1;
    }
    if (reset) {
        unsigned long long init[64];
        for (int i = 0; i < 64; ++i) init[i] = (i & 1) ? 0ull : ~0ull;
        if (cudaMemcpyToSymbol(g_timeline, init, sizeof(init)) != cudaSuccess) return -1;
    }
    return 0;
}
#endif

size_t stream_bf16_smem_bytes(int warps, int stages, int keys, int batch_for_tables) {
    size_t bytes = 1024;  // alignment slack
    bytes += (size_t)warps * stages * keys * 512;
    bytes += (size_t)warps * kHeadsPad * kOPitch * sizeof(float);
    bytes += 2 * (size_t)warps * kHeadsPad * sizeof(float);
    bytes += (size_t)warps * stages * sizeof(uint64_t);
    bytes += 2 * ((size_t)batch_for_tables + 1) * sizeof(int32_t);
    return bytes;
}

template <int WARPS, int STAGES, int KEYS, int OCC>
static cudaError_t launch_variant(const CUtensorMap& tk, const CUtensorMap& tv,
                                  const DecodeArgs& args, int grid, cudaStream_t stream) {
    const int tables = args.seq_lens_dev != nullptr ? args.batch : 0;
    const size_t smem = stream_bf16_smem_bytes(WARPS, STAGES, KEYS, tables);
    auto kernel = gqa_decode_stream_bf16<WARPS, STAGES, KEYS, OCC>;
    static size_t configured[64] = {};  // the attribute is per function and per device
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || configured[dev] < smem) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = smem;
    }
    return launch_pdl(kernel, dim3(grid), dim3(WARPS * 32), smem, stream, tk, tv, args);
}

cudaError_t launch_stream_bf16(const StreamShape& shape, const CUtensorMap& tk,
                               const CUtensorMap& tv, const DecodeArgs& args, int grid,
                               cudaStream_t stream) {
#define GQA_VARIANT(W, S, K, O)                                                     \
    if (shape.warps == W && shape.stages == S && shape.keys == K && shape.ctas_per_sm == O) { \
        return launch_variant<W, S, K, O>(tk, tv, args, grid, stream);               \
    }
    GQA_VARIANT(4, 1, 64, 1)
    GQA_VARIANT(4, 2, 32, 1)
    GQA_VARIANT(4, 3, 32, 1)
    GQA_VARIANT(8, 1, 32, 1)
    GQA_VARIANT(4, 1, 32, 2)
#undef GQA_VARIANT
    return cudaErrorInvalidValue;
}

}  // namespace gqa
