/*
 * CPU restatement of the inferrous-qwen3 W8A8 linear-layer arithmetic (plain C).
 * TEST INFRASTRUCTURE ONLY -- see w8a8_oracle.h for the parity status and the
 * reference file:line each function follows.
 *
 * Build: see oracle/Makefile (-O2 -ffp-contract=off: the reference compiles its
 * kernels with FMA contraction disabled, tools/cuda.sh:21, and uses explicit
 * round-to-nearest mul/add/div, src/kernels.rs:4-7).
 */
#include "w8a8_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

static inline uint32_t f2u(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    return u;
}
static inline float u2f(uint32_t u) {
    float x;
    memcpy(&x, &u, 4);
    return x;
}

/* src/kernels.rs:12-15 */
float oracle_bf16(float x) {
    uint32_t u = f2u(x);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    return u2f(u);
}
uint16_t oracle_bf16_bits(float x) { return (uint16_t)(f2u(oracle_bf16(x)) >> 16); }

/* src/kernels.rs:25-34.  Rust's f32::clamp keeps NaN; cvt.rni.s32.f32 turns NaN into 0. */
int8_t oracle_round_i8(float x) {
    if (x != x) return 0;
    if (x < -127.0f) x = -127.0f;
    if (x > 127.0f) x = 127.0f;
    /* nearbyintf under the default rounding mode is round-half-to-even. */
    return (int8_t)(int32_t)nearbyintf(x);
}
void oracle_round_i8_many(const float *x, int8_t *out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = oracle_round_i8(x[i]);
}

/* Rust f32::max / PTX max.f32: a NaN operand is ignored. */
static inline float max_ignoring_nan(float m, float v) { return (v > m) ? v : m; }

/* src/kernels.rs:433-451 */
void oracle_quantize(const float *x, int M, int K, int8_t *q, float *scale) {
    for (int r = 0; r < M; ++r) {
        const float *row = x + (size_t)r * K;
        float m = 1e-8f;
        for (int j = 0; j < K; ++j) m = max_ignoring_nan(m, fabsf(row[j]));
        volatile float s = m / 127.0f;
        scale[r] = s;
        for (int j = 0; j < K; ++j) {
            volatile float d = row[j] / s;
            q[(size_t)r * K + j] = oracle_round_i8(d);
        }
    }
}

/* src/kernels.rs:462-474 */
void oracle_quantize_with_max(const float *x, const uint32_t *maxima, int M, int K, int8_t *q,
                              float *scale) {
    for (int r = 0; r < M; ++r) {
        volatile float s = u2f(maxima[r]) / 127.0f;
        scale[r] = s;
        for (int j = 0; j < K; ++j) {
            volatile float d = x[(size_t)r * K + j] / s;
            q[(size_t)r * K + j] = oracle_round_i8(d);
        }
    }
}

/* src/kernels.rs:357-393 (generic width) == :508-547 (width 4096): same tree. */
void oracle_rmsnorm(const float *x, const float *gain, float eps, int M, int K, float *y) {
    for (int r = 0; r < M; ++r) {
        const float *row = x + (size_t)r * K;
        volatile float p[256];
        for (int t = 0; t < 256; ++t) {
            volatile float s = 0.0f;
            for (int j = t; j < K; j += 256) {
                volatile float sq = row[j] * row[j];
                s = s + sq;
            }
            p[t] = s;
        }
        for (int d = 128; d > 0; d /= 2)
            for (int t = 0; t < d; ++t) p[t] = p[t] + p[t + d];
        volatile float mean = p[0] / (float)K;
        volatile float arg = mean + eps;
        float inv = (float)(1.0 / sqrt((double)arg));
        for (int j = 0; j < K; ++j) {
            volatile float a = row[j] * inv;
            volatile float b = a * gain[j];
            y[(size_t)r * K + j] = oracle_bf16(b);
        }
    }
}

/* src/kernels.rs:2180-2181 (expression order), :134-147 (absmax on bit patterns). */
void oracle_swiglu(const float *gate, const float *up, size_t n, float *act, uint32_t *absmax_bits) {
    uint32_t best = f2u(1e-8f);
    for (size_t i = 0; i < n; ++i) {
        float g = gate[i];
        volatile float e = (float)exp(-(double)g);
        volatile float den = 1.0f + e;
        volatile float s = g / den;
        volatile float v = s * up[i];
        float a = oracle_bf16(v);
        act[i] = a;
        uint32_t bits = f2u(a) & 0x7fffffffu;
        if (bits > 0x7f800000u) bits = 0;
        if (bits > best) best = bits;
    }
    if (absmax_bits) *absmax_bits = best;
}

/* src/kernels.rs:2163-2170 */
void oracle_residual(const float *a, const float *b, size_t n, float *out) {
    for (size_t i = 0; i < n; ++i) {
        volatile float s = a[i] + b[i];
        out[i] = oracle_bf16(s);
    }
}

/* One int8 x int8 dot product, int32 accumulation.  |sum| <= 12288*127^2 < 2^31
 * (docs/qwen3-8b-w8a8/safety.md:34), so any summation order gives the same bits.
 * Function multiversioning lets one binary use AVX2 / AVX-512 where the host has them. */
#if defined(__x86_64__) && defined(__GNUC__) && !defined(ORACLE_NO_CLONES)
__attribute__((target_clones("default", "avx2", "arch=x86-64-v4")))
#endif
static int32_t dot_i8(const int8_t *a, const int8_t *b, int K) {
    int32_t acc = 0;
    for (int k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
    return acc;
}

int oracle_hw_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

struct acc_job {
    const int8_t *q, *w;
    int M, N, K, n0, n1;
    int32_t *acc;
};

static void *acc_worker(void *arg) {
    const struct acc_job *j = (const struct acc_job *)arg;
    for (int n = j->n0; n < j->n1; ++n) {
        const int8_t *wr = j->w + (size_t)n * j->K;
        for (int m = 0; m < j->M; ++m)
            j->acc[(size_t)m * j->N + n] = dot_i8(j->q + (size_t)m * j->K, wr, j->K);
    }
    return NULL;
}

/* src/kernels.rs:280-289; tools/operator_fixtures.py:54 (q.int() @ w.int().T).
 * Output channels are split evenly over `threads` POSIX threads. */
void oracle_linear_acc(const int8_t *q, const int8_t *w, int M, int N, int K, int32_t *acc,
                       int threads) {
    if (threads <= 0) threads = oracle_hw_threads();
    if (threads > N) threads = N > 0 ? N : 1;
    if (threads > 256) threads = 256;
    struct acc_job jobs[256];
    pthread_t tid[256];
    int per = (N + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        int n0 = t * per, n1 = n0 + per > N ? N : n0 + per;
        if (n0 > N) n0 = N;
        jobs[t] = (struct acc_job){q, w, M, N, K, n0, n1, acc};
    }
    for (int t = 1; t < threads; ++t) pthread_create(&tid[t], NULL, acc_worker, &jobs[t]);
    acc_worker(&jobs[0]);
    for (int t = 1; t < threads; ++t) pthread_join(tid[t], NULL);
}

/* src/kernels.rs:290 */
void oracle_epilogue(const int32_t *acc, const float *asc, const float *ws, int M, int N, float *y) {
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            volatile float a = (float)acc[(size_t)m * N + n]; /* cvt.rn.f32.s32 */
            volatile float b = a * asc[m];
            volatile float c = b * ws[n];
            y[(size_t)m * N + n] = oracle_bf16(c);
        }
}

void oracle_linear(const int8_t *q, const float *asc, const int8_t *w, const float *ws, int M, int N,
                   int K, const float *residual, float *y, float *combined, int threads) {
    int32_t *acc = (int32_t *)malloc((size_t)M * N * sizeof(int32_t));
    oracle_linear_acc(q, w, M, N, K, acc, threads);
    oracle_epilogue(acc, asc, ws, M, N, y);
    free(acc);
    /* src/kernels.rs:612-616 */
    if (residual && combined) oracle_residual(residual, y, (size_t)M * N, combined);
}

/* tools/prepare.py:79-81 */
void oracle_weight_quantize(const float *w, int N, int K, int8_t *q, float *scale) {
    oracle_quantize(w, N, K, q, scale);
}
