/*
 * CPU oracle for Qwen3 decode-phase grouped-query attention and its front stage.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the arithmetic of the
 * reference engine's attention path so that the CUDA kernels can be checked against it and
 * so that a CPU baseline can be timed. It is never linked into, loaded by, or used as a
 * fallback for the product library.
 *
 * Parity status: the reference ships no golden vectors for attention; its CPU attention
 * cannot be built (Armadillo, glog) and has its score computation commented out. The
 * restatement is therefore pinned against outputs of the reference's own CUDA kernels run
 * on a B200 (tests/golden/, produced by tests/golden/make_golden.py from
 * oracle/_ref/libref_attn.so), not against a reference test fixture.
 *
 * What each function follows (paths inside the reference project):
 *   oracle_gqa_decode        code/source/op/kernel/cpu/mha_kernel.cpp:34-110 (loop structure,
 *                            cache indexing, scale = 1/sqrtf(head_dim)); the score it no
 *                            longer computes (:75, commented out) is restored as
 *                            scale * dot(q_h, K_t), which is what the commented call and
 *                            cpu/matmul_kernel.cpp:48-51 compute; softmax as
 *                            cpu/softmax_kernel.cpp:11-19 (subtract max, exp, divide by the
 *                            sum); weighted V sum in key order as
 *                            cpu/scale_sum_kernel.cpp:29-35.
 *   oracle_mha_kernel_cpu    the same, behind the reference's CPU kernel argument list
 *                            (cpu/mha_kernel.cpp:6-20) with its 32-bit offsets.
 *   oracle_qk_norm_rope      code/source/op/kernel/cuda/rmsnorm_kernel.cu:221-244 and the
 *                            Python restatement test_kernel/test_qwen3_bf16_ops.py:777-794.
 *   oracle_sin_cos_cache     code/source/op/kernel/cpu/rope_kernel.cpp:5-23 (form 0) and
 *                            code/source/op/kernel/cuda/rope_kernel.cu:6-21 (form 1).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_DTYPE_F32 0
#define ORACLE_DTYPE_BF16 1

static inline float bf16_bits_to_f32(uint16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

/* Round to nearest even, NaN kept quiet: what __float2bfloat16 does on the device. */
static inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
        return (uint16_t)0x7fffu;
    }
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

void oracle_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16_bits(src[i]);
}

void oracle_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = bf16_bits_to_f32(src[i]);
}

/* Number of threads for the parallel loops (launchers like torchrun export OMP_NUM_THREADS=1). */
void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

static inline float load_elem(const void* base, int dtype, int64_t idx) {
    if (dtype == ORACLE_DTYPE_F32) return ((const float*)base)[idx];
    return bf16_bits_to_f32(((const uint16_t*)base)[idx]);
}

/* Widens one cache row of d channels to FP32 (a copy for FP32 storage). */
static inline void load_row(const void* base, int dtype, int64_t off, int d, float* dst) {
    if (dtype == ORACLE_DTYPE_F32) {
        memcpy(dst, (const float*)base + off, sizeof(float) * (size_t)d);
    } else {
        const uint16_t* src = (const uint16_t*)base + off;
        for (int i = 0; i < d; ++i) dst[i] = bf16_bits_to_f32(src[i]);
    }
}

/*
 * One (sequence, query head): scores, softmax, weighted sum, FP32 accumulation in the
 * reference's order (keys ascending, channels ascending).
 */
static void head_f32(const void* q, const void* kc, const void* vc, int dtype, int64_t q_off,
                     int d, int len, const int64_t* row_off, float* score, float* out) {
    const float scale = 1.0f / sqrtf((float)d);
    float qf[512];
    float row[512];
    for (int i = 0; i < d; ++i) qf[i] = load_elem(q, dtype, q_off + i);
    for (int t = 0; t < len; ++t) {
        float acc = 0.0f;
        load_row(kc, dtype, row_off[t], d, row);
        for (int i = 0; i < d; ++i) acc += qf[i] * row[i];
        score[t] = acc * scale;
    }
    float mx = score[0];
    for (int t = 1; t < len; ++t) mx = score[t] > mx ? score[t] : mx;
    float sum = 0.0f;
    for (int t = 0; t < len; ++t) {
        score[t] = expf(score[t] - mx);
        sum += score[t];
    }
    for (int t = 0; t < len; ++t) score[t] /= sum;
    for (int i = 0; i < d; ++i) out[i] = 0.0f;
    for (int t = 0; t < len; ++t) {
        const float p = score[t];
        load_row(vc, dtype, row_off[t], d, row);
        for (int i = 0; i < d; ++i) out[i] += p * row[i];
    }
}

/* The same in FP64: ground truth for error measurement. */
static void head_f64(const void* q, const void* kc, const void* vc, int dtype, int64_t q_off,
                     int d, int len, const int64_t* row_off, double* score, float* out) {
    const double scale = 1.0 / sqrt((double)d);
    double qf[512];
    double acc_out[512];
    float row[512];
    for (int i = 0; i < d; ++i) qf[i] = (double)load_elem(q, dtype, q_off + i);
    double mx = -INFINITY;
    for (int t = 0; t < len; ++t) {
        double acc = 0.0;
        load_row(kc, dtype, row_off[t], d, row);
        for (int i = 0; i < d; ++i) acc += qf[i] * (double)row[i];
        score[t] = acc * scale;
        mx = score[t] > mx ? score[t] : mx;
    }
    double sum = 0.0;
    for (int t = 0; t < len; ++t) {
        score[t] = exp(score[t] - mx);
        sum += score[t];
    }
    for (int i = 0; i < d; ++i) acc_out[i] = 0.0;
    for (int t = 0; t < len; ++t) {
        const double p = score[t] / sum;
        load_row(vc, dtype, row_off[t], d, row);
        for (int i = 0; i < d; ++i) acc_out[i] += p * (double)row[i];
    }
    for (int i = 0; i < d; ++i) out[i] = (float)acc_out[i];
}

/*
 * Batched GQA decode attention over a strided, optionally paged KV cache.
 *
 *   q        [batch, hq, d]              dtype f32 or bf16 bits
 *   k, v     element (b, t, hk, i) lives at
 *              blk(b, t) * stride_blk + (t % block_tokens) * stride_tok + hk * stride_head + i
 *            where blk(b, t) = block_table[b * blocks_per_seq + t / block_tokens] when a
 *            block table is given, else `fixed_block` (the reference's layer_id; its layout
 *            is stride_blk = max_seq_len * kv_dim, stride_tok = kv_dim, stride_head = d,
 *            block_tokens = max_seq_len).
 *   seq_lens [batch]   number of cached positions attended (pos + 1); all are attended.
 *   out      [batch, hq, d] FP32 (not rounded; the caller rounds when comparing BF16).
 *   accum    0 = FP32 in the reference's order, 1 = FP64.
 *   threads  <= 0: all cores.  The reference loops heads on one thread; the threaded form
 *            is for the all-cores baseline and gives the same values (heads are independent).
 * Returns 0, or -1 on a bad argument.
 */
int oracle_gqa_decode(const void* q, const void* k, const void* v, float* out, int dtype,
                      int accum, int batch, int hq, int hkv, int d, const int32_t* seq_lens,
                      int64_t stride_blk, int64_t stride_tok, int64_t stride_head,
                      int32_t block_tokens, const int32_t* block_table, int32_t blocks_per_seq,
                      int32_t fixed_block, int threads) {
    if (!q || !k || !v || !out || !seq_lens) return -1;
    if (batch <= 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || d <= 0 || d > 512) return -1;
    if (block_tokens <= 0) return -1;
    if (dtype != ORACLE_DTYPE_F32 && dtype != ORACLE_DTYPE_BF16) return -1;
    const int kv_mul = hq / hkv;
    int max_len = 0;
    for (int b = 0; b < batch; ++b) {
        if (seq_lens[b] <= 0) return -1;
        if (seq_lens[b] > max_len) max_len = seq_lens[b];
    }
#ifdef _OPENMP
    const int nthreads = threads > 0 ? threads : omp_get_max_threads();
#else
    const int nthreads = 1;
    (void)threads;
#endif
    int failed = 0;
#pragma omp parallel num_threads(nthreads)
    {
        int64_t* row_off = (int64_t*)malloc(sizeof(int64_t) * (size_t)max_len);
        void* score = malloc(sizeof(double) * (size_t)max_len);
        if (!row_off || !score) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for collapse(2) schedule(dynamic, 1)
            for (int b = 0; b < batch; ++b) {
                for (int h = 0; h < hq; ++h) {
                    const int len = seq_lens[b];
                    const int hk = h / kv_mul;
                    for (int t = 0; t < len; ++t) {
                        const int64_t blk =
                            block_table
                                ? (int64_t)block_table[(int64_t)b * blocks_per_seq + t / block_tokens]
                                : (int64_t)fixed_block;
                        row_off[t] = blk * stride_blk + (int64_t)(t % block_tokens) * stride_tok +
                                     (int64_t)hk * stride_head;
                    }
                    const int64_t q_off = ((int64_t)b * hq + h) * d;
                    float* o = out + q_off;
                    if (accum == 0) {
                        head_f32(q, k, v, dtype, q_off, d, len, row_off, (float*)score, o);
                    } else {
                        head_f64(q, k, v, dtype, q_off, d, len, row_off, (double*)score, o);
                    }
                }
            }
        }
        free(row_off);
        free(score);
    }
    return failed ? -1 : 0;
}

/*
 * The reference's CPU kernel argument list (FP32 tensors, one sequence, cache
 * [layer, max_seq_len, kv_dim]); `score` is its [head_num, max_seq_len] scratch and is left
 * holding the softmax probabilities of each head, as the reference leaves it.
 */
int oracle_mha_kernel_cpu(const float* query, float* score, const float* key_cache,
                          const float* value_cache, float* output, int32_t layer_id, int32_t pos,
                          int32_t kv_dim, int32_t kv_mul, int32_t head_num, int32_t head_dim,
                          int32_t max_seq_len) {
    if (!query || !score || !key_cache || !value_cache || !output) return -1;
    if (pos < 0 || pos >= max_seq_len || head_dim <= 0 || head_dim > 512 || kv_mul <= 0) return -1;
    const int32_t layer_offset = layer_id * max_seq_len * kv_dim;
    const int len = pos + 1;
    int64_t* row_off = (int64_t*)malloc(sizeof(int64_t) * (size_t)len);
    if (!row_off) return -1;
    for (int32_t h = 0; h < head_num; ++h) {
        for (int t = 0; t < len; ++t) {
            row_off[t] = (int64_t)(layer_offset + t * kv_dim + (h / kv_mul) * head_dim);
        }
        head_f32(query, key_cache, value_cache, ORACLE_DTYPE_F32, (int64_t)h * head_dim, head_dim,
                 len, row_off, score + (int64_t)h * max_seq_len, output + (int64_t)h * head_dim);
    }
    free(row_off);
    return 0;
}

/*
 * Per-head RMSNorm * weight then rotate-half RoPE with the given sin/cos row, for `heads`
 * heads of `d` channels. x, w: bf16 bits; out: bf16 bits (may alias x). FP32 math with one
 * rounding at the end; accum 1 computes the mean square in FP64.
 */
static void norm_rope_heads(const uint16_t* x, const uint16_t* w, const float* sin_row,
                            const float* cos_row, int heads, int d, float eps, int accum,
                            uint16_t* out) {
    const int half = d / 2;
    for (int h = 0; h < heads; ++h) {
        const uint16_t* xi = x + (int64_t)h * d;
        uint16_t* oi = out + (int64_t)h * d;
        float s;
        if (accum == 0) {
            float sum = 0.0f;
            for (int i = 0; i < d; ++i) {
                const float val = bf16_bits_to_f32(xi[i]);
                sum += val * val;
            }
            s = 1.0f / sqrtf(sum / (float)d + eps);
        } else {
            double sum = 0.0;
            for (int i = 0; i < d; ++i) {
                const double val = (double)bf16_bits_to_f32(xi[i]);
                sum += val * val;
            }
            s = (float)(1.0 / sqrt(sum / (double)d + (double)eps));
        }
        for (int i = 0; i < half; ++i) {
            const float a = bf16_bits_to_f32(xi[i]) * bf16_bits_to_f32(w[i]) * s;
            const float b = bf16_bits_to_f32(xi[i + half]) * bf16_bits_to_f32(w[i + half]) * s;
            const float sn = sin_row[i];
            const float cs = cos_row[i];
            const float a1 = a * cs - b * sn;
            const float b1 = a * sn + b * cs;
            oi[i] = f32_to_bf16_bits(a1);
            oi[i + half] = f32_to_bf16_bits(b1);
        }
    }
}

/*
 * query [hq * d] and key [hkv * d] are normalised and rotated in place; weight is
 * [2 * d] = q_norm then k_norm; sin_row / cos_row are the [d / 2] table rows of the token's
 * position.
 */
int oracle_qk_norm_rope(uint16_t* query, uint16_t* key, const uint16_t* weight,
                        const float* sin_row, const float* cos_row, int hq, int hkv, int d,
                        float eps, int accum) {
    if (!query || !key || !weight || !sin_row || !cos_row || d <= 0 || (d & 1)) return -1;
    norm_rope_heads(query, weight, sin_row, cos_row, hq, d, eps, accum, query);
    norm_rope_heads(key, weight + d, sin_row, cos_row, hkv, d, eps, accum, key);
    return 0;
}

/*
 * sin/cos tables [max_seq_len, d / 2], FP32.
 *   form 0: the reference's CPU form, freq_i = (float)exp(-2.0 * i * (1/d) * ln(1e6)).
 *   form 1: the reference's CUDA form, freq_i = 1 / powf(1e6, 2i / d).
 * Both then take sinf/cosf of (float)pos * freq_i.
 */
int oracle_sin_cos_cache(float* sin_cache, float* cos_cache, int d, int max_seq_len, int form) {
    if (!sin_cache || !cos_cache || d <= 0 || (d & 1) || max_seq_len <= 0) return -1;
    const int half = d / 2;
    float* freq = (float*)malloc(sizeof(float) * (size_t)half);
    if (!freq) return -1;
    const float inv_d = 1.0f / (float)d;
    const float ln_base = logf(1000000.0f);
    for (int i = 0; i < half; ++i) {
        if (form == 0) {
            freq[i] = (float)exp(-2.0 * i * inv_d * ln_base);
        } else {
            freq[i] = 1.0f / powf(1000000.0f, (2.0f * (float)i) / (float)d);
        }
    }
    for (int pos = 0; pos < max_seq_len; ++pos) {
        for (int i = 0; i < half; ++i) {
            const float theta = (float)pos * freq[i];
            sin_cache[(int64_t)pos * half + i] = sinf(theta);
            cos_cache[(int64_t)pos * half + i] = cosf(theta);
        }
    }
    free(freq);
    return 0;
}
