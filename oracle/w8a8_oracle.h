/*
 * CPU restatement of the inferrous-qwen3 W8A8 linear-layer arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product library links, loads or
 * calls this file; it exists so that the CUDA path can be checked against an
 * independent plain-C statement of what the reference computes, and so that a
 * CPU baseline can be timed beside the GPU.
 *
 * Parity status: PINNED for quantize / linear / residual (bit-exact against the
 * reference's own PyTorch-CPU fixture generator, tools/operator_fixtures.py,
 * whose outputs are committed under tests/golden/operator_fixtures/).
 * rmsnorm and swiglu are pinned to those fixtures only within the reference's
 * numeric gate (|err| <= 2e-4 + 0.01*|expected|, docs/qwen3-8b-w8a8/coverage.md:28),
 * because the reference computes them with hardware approximations
 * (rsqrt.approx, ex2.approx) whose bit patterns no fixture holds.
 *
 * Every function cites the reference file:line it follows
 * (paths relative to crates/inferrous-qwen3/).
 */
#ifndef W8A8_ORACLE_H
#define W8A8_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* src/kernels.rs:12-15  f32 -> nearest-even bf16, kept as f32 (no NaN special case). */
float oracle_bf16(float x);
/* bf16 bit pattern (upper 16 bits of oracle_bf16). */
uint16_t oracle_bf16_bits(float x);
/* src/kernels.rs:25-34  clamp(+-127) then round-to-nearest-even; NaN -> 0. */
int8_t oracle_round_i8(float x);
void oracle_round_i8_many(const float *x, int8_t *out, size_t n);

/* src/kernels.rs:415-452, tools/operator_fixtures.py:43-44.
 * m = max(1e-8, max_j |x[r,j]|) ignoring NaN; scale[r] = m/127; q = round(x/scale). */
void oracle_quantize(const float *x, int M, int K, int8_t *q, float *scale);
/* src/kernels.rs:455-475: same with the row maximum given as f32 bit patterns. */
void oracle_quantize_with_max(const float *x, const uint32_t *maxima, int M, int K,
                              int8_t *q, float *scale);

/* src/kernels.rs:347-413 and :479-576.  Sum of squares with the reference's tree
 * (256 partials of K/256 strided terms, then distances 128..1), non-fused
 * multiply/add; inv = 1/sqrt(ss/K + eps) correctly rounded (the reference uses
 * rsqrt.approx); y = bf16((x*inv)*gain). */
void oracle_rmsnorm(const float *x, const float *gain, float eps, int M, int K, float *y);

/* src/kernels.rs:2172-2190: act = bf16((g / (1 + exp(-g))) * u); exp evaluated in
 * double and rounded (the reference uses ex2.approx).  absmax_bits (optional)
 * receives max over the row of |act| as f32 bits, floor 1e-8, NaN ignored
 * (src/kernels.rs:134-147). */
void oracle_swiglu(const float *gate, const float *up, size_t n, float *act, uint32_t *absmax_bits);

/* src/kernels.rs:2163-2170: bf16(a + b). */
void oracle_residual(const float *a, const float *b, size_t n, float *out);

/* src/kernels.rs:270-289, tools/operator_fixtures.py:54: acc[m,n] = sum_k q[m,k]*w[n,k] in int32.
 * threads <= 0 means "all host threads". */
void oracle_linear_acc(const int8_t *q, const int8_t *w, int M, int N, int K, int32_t *acc,
                       int threads);
/* src/kernels.rs:290: y = bf16((f32(acc) * asc[m]) * ws[n]); two separately rounded multiplies. */
void oracle_epilogue(const int32_t *acc, const float *asc, const float *ws, int M, int N, float *y);
/* oracle_linear_acc + oracle_epilogue; residual/combined optional (src/kernels.rs:612-616:
 * combined = bf16(residual + y), y rounded first). */
void oracle_linear(const int8_t *q, const float *asc, const int8_t *w, const float *ws, int M, int N,
                   int K, const float *residual, float *y, float *combined, int threads);

/* tools/prepare.py:79-81: scale[n] = max(1e-8, max_k |w[n,k]|)/127; q = round_half_even(w/scale) clamp +-127. */
void oracle_weight_quantize(const float *w, int N, int K, int8_t *q, float *scale);

int oracle_hw_threads(void);

#ifdef __cplusplus
}
#endif
#endif
