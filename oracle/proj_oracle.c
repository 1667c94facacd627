/*
 * CPU oracle for the two projections that sit on either side of decode attention: the
 * packed QKV GEMV in front of it and the output projection with residual add behind it.
 *
 * TEST INFRASTRUCTURE ONLY, like gqa_oracle.c: never linked into, loaded by, or used as a
 * fallback for the product library.
 *
 * Parity status: pinned. With accum = 0 the functions restate the reference's CUDA kernels
 * operation by operation (the per-thread strided FMA chain of 256 threads, the shuffle tree
 * inside each warp, the tree over the 8 warp sums), so their results are bit-equal to the
 * outputs of the reference's own kernels stored in tests/golden/ref_cuda_proj.npz. With
 * accum = 1 the dot products are taken in FP64 (ground truth for tolerance checks).
 *
 * What each function follows (paths inside the reference project):
 *   oracle_gemv_add   fused_gemv_add_bf16x8_kernel  code/source/op/kernel/cuda/matmul_kernel.cu:143-170
 *                     (residual[n] = bf16(float(residual[n]) + dot(in, W[n])))
 *   oracle_qkv_gemv   fused_qkv_gemv_bf16x8_kernel  code/source/op/kernel/cuda/matmul_kernel.cu:211-245
 *                     (rows [0, dim) -> query, [dim, dim + kv_dim) -> key, the rest -> value)
 *   block sum         warp_reduce_sum / block_reduce_sum  matmul_kernel.cu:6-36
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define REF_THREADS 256

static inline float bits_to_f32(uint16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

static inline uint16_t f32_to_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)0x7fffu;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* dot(x, w) over k elements in the reference kernel's order (k % 8 == 0). */
static float dot_reference_order(const uint16_t* x, const uint16_t* w, int k) {
    float part[REF_THREADS];
    const int k8 = k / 8;
    for (int t = 0; t < REF_THREADS; ++t) {
        float sum = 0.0f;
        for (int i = t; i < k8; i += REF_THREADS) {
            for (int j = 0; j < 8; ++j) {
                /* nvcc contracts `sum += a * b` into one fused multiply-add */
                sum = fmaf(bits_to_f32(x[8 * i + j]), bits_to_f32(w[8 * i + j]), sum);
            }
        }
        part[t] = sum;
    }
    /* shuffle-down tree inside each warp: only lane 0's value is used afterwards */
    float warp_sum[REF_THREADS / 32];
    for (int wp = 0; wp < REF_THREADS / 32; ++wp) {
        float v[32];
        memcpy(v, part + 32 * wp, sizeof v);
        for (int delta = 16; delta > 0; delta >>= 1) {
            for (int lane = 0; lane + delta < 32; ++lane) v[lane] += v[lane + delta];
        }
        warp_sum[wp] = v[0];
    }
    /* the same tree, 8 wide, over the warp sums */
    for (int delta = 4; delta > 0; delta >>= 1) {
        for (int lane = 0; lane + delta < 8; ++lane) warp_sum[lane] += warp_sum[lane + delta];
    }
    return warp_sum[0];
}

static double dot_f64(const uint16_t* x, const uint16_t* w, int k) {
    double sum = 0.0;
    for (int i = 0; i < k; ++i) sum += (double)bits_to_f32(x[i]) * (double)bits_to_f32(w[i]);
    return sum;
}

/*
 * residual [batch, n] += x [batch, k] . weight[n, ld]^T, BF16 bits in and out. `ld` is the
 * element pitch between weight rows (>= k). With accum = 2 the FP64 sums are returned
 * unrounded in out_f64 [batch, n] (residual included) and `residual` is left alone.
 */
int oracle_gemv_add(const uint16_t* x, const uint16_t* weight, uint16_t* residual, double* out_f64,
                    int batch, int n, int k, int64_t ld, int accum) {
    if (!x || !weight || !residual || batch <= 0 || n <= 0 || k <= 0 || (k % 8) || ld < k) {
        return -1;
    }
    if (accum == 2 && !out_f64) return -1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
        for (int row = 0; row < n; ++row) {
            const uint16_t* xr = x + (int64_t)b * k;
            const uint16_t* wr = weight + (int64_t)row * ld;
            uint16_t* r = residual + (int64_t)b * n + row;
            if (accum == 0) {
                *r = f32_to_bits(bits_to_f32(*r) + dot_reference_order(xr, wr, k));
            } else if (accum == 1) {
                *r = f32_to_bits((float)((double)bits_to_f32(*r) + dot_f64(xr, wr, k)));
            } else {
                out_f64[(int64_t)b * n + row] = (double)bits_to_f32(*r) + dot_f64(xr, wr, k);
            }
        }
    }
    return 0;
}

/*
 * x [batch, hidden]; weight [dim + 2 * kv_dim, hidden]; query [batch, dim], key and value
 * [batch, kv_dim], all BF16 bits.
 */
int oracle_qkv_gemv(const uint16_t* x, const uint16_t* weight, uint16_t* query, uint16_t* key,
                    uint16_t* value, int batch, int hidden, int dim, int kv_dim, int accum) {
    if (!x || !weight || !query || !key || !value || batch <= 0 || hidden <= 0 || (hidden % 8) ||
        dim <= 0 || kv_dim <= 0) {
        return -1;
    }
    const int rows = dim + 2 * kv_dim;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
        for (int row = 0; row < rows; ++row) {
            const uint16_t* xr = x + (int64_t)b * hidden;
            const uint16_t* wr = weight + (int64_t)row * hidden;
            const float sum = accum == 0 ? dot_reference_order(xr, wr, hidden)
                                         : (float)dot_f64(xr, wr, hidden);
            const uint16_t bits = f32_to_bits(sum);
            if (row < dim) {
                query[(int64_t)b * dim + row] = bits;
            } else if (row < dim + kv_dim) {
                key[(int64_t)b * kv_dim + row - dim] = bits;
            } else {
                value[(int64_t)b * kv_dim + row - dim - kv_dim] = bits;
            }
        }
    }
    return 0;
}
