// The reference's own output head: bf16 weights [vocab, hidden], float32 accumulation, bf16 logits
// (crates/inferrous-qwen3/src/kernels.rs: `head` :2233-2257; `head_packed` :2259-2373 computes the same bits from a
// 12-bit packed copy of the weights; launched at src/gpu.rs:801-809, selection `select_token` :2191-2231 at :811).
// The checkpoint exporter leaves the head unquantized (tools/prepare.py:99: "ignore": ["lm_head"]), so a host that runs
// a real bundle needs this kernel to reproduce the reference's logits; the W8A8 head (w8a8_linear_argmax) is the
// benchmark's projection shape, not the reference's arithmetic.
//
// The float32 sum is not associative, so the kernel keeps the reference's order exactly: lane L of a warp adds the
// products of columns L, L + 32, L + 64, ... in that order (separately rounded multiply and add), then the 32 partial
// sums meet in a shuffle-down tree of distances 16, 8, 4, 2, 1; the logit is bf16(sum).  The result is bit-identical to
// `head` / `head_packed` on the same inputs.
// What differs is who computes which partial sum.  The order only fixes how each of the 32 partial sums of a row is built
// and how they are added up, not which thread holds them: here four threads share a row, each loads 16 bytes (eight
// consecutive columns) per step of 32 columns and keeps the eight partial sums of those columns in registers, so a warp
// works on eight rows per load instruction; the tree over the 32 partial sums is two exchanges between the four threads
// and three levels inside a thread.  (One two-byte load per element and lane, the direct transcription, is bound by
// instruction issue: 57.8 % of the issue slots and 43 % of the load/store pipe busy at 4.5 TB/s; widths that are not a
// multiple of 32 still take that form.)  The activation row is parked in shared memory once per CTA, and the greedy
// selection is fused in: a CTA of 8 warps leaves the best
// (value, index) of its 16 rows as one packed key, which the reduction kernel of the W8A8 head finishes
// (launch_argmax_finish), so the 151 936 logits need not be written.  Bound by the 1.24 GB stream of weights from HBM.
#include "../../include/qwen3_glue.h"
#include "../../include/w8a8.h"
#include "common.cuh"
#include "internal.h"

namespace w8a8 {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerCta = 16;  // two per warp; the candidate buffer holds one slot of 16 keys per CTA
constexpr int kUnroll = 16;

__device__ __forceinline__ uint32_t ld_stream_u16(const uint16_t *p) {
    uint16_t r;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
}

template <class T>
__global__ void __launch_bounds__(kThreads) head_bf16_kernel(const typename T::storage *__restrict__ x, const uint16_t *__restrict__ w,
                                                             int K, int vocab, typename T::storage *__restrict__ logits,
                                                             unsigned long long *__restrict__ partial_best) {
    extern __shared__ __align__(16) float xs[];  // [K]
    __shared__ unsigned long long cand[kRowsPerCta];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r0 = blockIdx.x * kRowsPerCta + 2 * warp;
    const uint16_t *w0 = w + (size_t)min(r0, vocab - 1) * K + lane;       // rows beyond the vocabulary are computed and dropped
    const uint16_t *w1 = w + (size_t)min(r0 + 1, vocab - 1) * K + lane;
    uint32_t a[kUnroll], b[kUnroll];
    // the first batch of weights does not depend on the preceding kernel
#pragma unroll
    for (int i = 0; i < kUnroll; ++i) {
        const int j = 32 * i + lane;
        a[i] = j < K ? ld_stream_u16(w0 + 32 * i) : 0u;
        b[i] = j < K ? ld_stream_u16(w1 + 32 * i) : 0u;
    }
    dependency_wait();
    for (int j = tid; j < K; j += kThreads) xs[j] = T::load(x + j);
    __syncthreads();
    float s0 = 0.0f, s1 = 0.0f;
    for (int base = 0; base < K; base += 32 * kUnroll) {
        float xv[kUnroll];
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
            const int j = base + 32 * i + lane;
            xv[i] = j < K ? xs[j] : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) {
            if (base + 32 * i + lane < K) {  // lane-strided, in column order (src/kernels.rs:2245-2249)
                s0 = __fadd_rn(s0, __fmul_rn(xv[i], __uint_as_float(a[i] << 16)));
                s1 = __fadd_rn(s1, __fmul_rn(xv[i], __uint_as_float(b[i] << 16)));
            }
        }
        const int next = base + 32 * kUnroll;
        if (next < K) {
#pragma unroll
            for (int i = 0; i < kUnroll; ++i) {
                const int j = next + 32 * i + lane;
                a[i] = j < K ? ld_stream_u16(w0 + next + 32 * i) : 0u;
                b[i] = j < K ? ld_stream_u16(w1 + next + 32 * i) : 0u;
            }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {  // src/kernels.rs:2250-2253
        s0 = __fadd_rn(s0, __shfl_down_sync(0xffffffffu, s0, d));
        s1 = __fadd_rn(s1, __shfl_down_sync(0xffffffffu, s1, d));
    }
    if (lane == 0) {
        const float v0 = bf16_rne(s0), v1 = bf16_rne(s1);
        if (logits) {
            if (r0 < vocab) T::store(logits + r0, v0);
            if (r0 + 1 < vocab) T::store(logits + r0 + 1, v1);
        }
        cand[2 * warp] = r0 < vocab ? argmax_key(v0, (uint32_t)r0) : 0ull;
        cand[2 * warp + 1] = r0 + 1 < vocab ? argmax_key(v1, (uint32_t)(r0 + 1)) : 0ull;
    }
    if (partial_best == nullptr) return;
    __syncthreads();
    if (tid < 16) {  // slot layout of the W8A8 head's candidates: 16 keys per CTA, key 0 = the one row of activations
        unsigned long long best = 0;
        if (tid == 0) {
#pragma unroll
            for (int r = 0; r < kRowsPerCta; ++r) best = max(best, cand[r]);
        }
        partial_best[(size_t)blockIdx.x * 16 + tid] = best;
    }
}

// K % 32 == 0, w 16-byte aligned: four threads per row (quad lane q holds the partial sums of columns 8 q .. 8 q + 7 of
// every 32-column step), eight rows per warp, 64 per CTA.
constexpr int kQuadRowsPerCta = 64;
constexpr int kQuadLoads = 8;  // 16-byte loads in flight per thread

template <class T>
__global__ void __launch_bounds__(kThreads) head_bf16_quad_kernel(const typename T::storage *__restrict__ x, const uint16_t *__restrict__ w,
                                                                  int K, int vocab, typename T::storage *__restrict__ logits,
                                                                  unsigned long long *__restrict__ partial_best) {
    extern __shared__ __align__(16) float xs[];  // [K]
    __shared__ unsigned long long cand[kQuadRowsPerCta];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q = lane & 3, in_warp = lane >> 2;
    const int local = warp * 8 + in_warp;
    const int row = blockIdx.x * kQuadRowsPerCta + local;
    const uint16_t *wr = w + (size_t)min(row, vocab - 1) * K + 8 * q;  // rows beyond the vocabulary are computed and dropped
    const int steps = K / 32;
    uint4 v[kQuadLoads];
    auto issue = [&](int first) {
#pragma unroll
        for (int u = 0; u < kQuadLoads; ++u) v[u] = first + u < steps ? ld_stream_16(wr + 32 * (first + u)) : make_uint4(0, 0, 0, 0);
    };
    issue(0);  // the first batch of weights does not depend on the preceding kernel
    dependency_wait();
    for (int j = tid; j < K; j += kThreads) xs[j] = T::load(x + j);
    __syncthreads();
    float p[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    for (int first = 0; first < steps; first += kQuadLoads) {
#pragma unroll
        for (int u = 0; u < kQuadLoads; ++u) {
            if (first + u < steps) {  // partial sum of column c: products of c, c + 32, ... in that order (src/kernels.rs:2245-2249)
                const float4 xa = *reinterpret_cast<const float4 *>(xs + 32 * (first + u) + 8 * q);
                const float4 xb = *reinterpret_cast<const float4 *>(xs + 32 * (first + u) + 8 * q + 4);
                p[0] = __fadd_rn(p[0], __fmul_rn(xa.x, __uint_as_float(v[u].x << 16)));
                p[1] = __fadd_rn(p[1], __fmul_rn(xa.y, __uint_as_float(v[u].x & 0xffff0000u)));
                p[2] = __fadd_rn(p[2], __fmul_rn(xa.z, __uint_as_float(v[u].y << 16)));
                p[3] = __fadd_rn(p[3], __fmul_rn(xa.w, __uint_as_float(v[u].y & 0xffff0000u)));
                p[4] = __fadd_rn(p[4], __fmul_rn(xb.x, __uint_as_float(v[u].z << 16)));
                p[5] = __fadd_rn(p[5], __fmul_rn(xb.y, __uint_as_float(v[u].z & 0xffff0000u)));
                p[6] = __fadd_rn(p[6], __fmul_rn(xb.z, __uint_as_float(v[u].w << 16)));
                p[7] = __fadd_rn(p[7], __fmul_rn(xb.w, __uint_as_float(v[u].w & 0xffff0000u)));
            }
        }
        if (first + kQuadLoads < steps) issue(first + kQuadLoads);
    }
    // the reference's tree over the 32 partial sums P[0..31] (src/kernels.rs:2250-2253): distances 16 and 8 pair
    // partial sums of different quad lanes (q ^ 2, then q ^ 1), distances 4, 2, 1 pair sums inside quad lane 0
#pragma unroll
    for (int k = 0; k < 8; ++k) p[k] = __fadd_rn(p[k], __shfl_xor_sync(0xffffffffu, p[k], 2));
#pragma unroll
    for (int k = 0; k < 8; ++k) p[k] = __fadd_rn(p[k], __shfl_xor_sync(0xffffffffu, p[k], 1));
    const float c0 = __fadd_rn(p[0], p[4]), c1 = __fadd_rn(p[1], p[5]), c2 = __fadd_rn(p[2], p[6]), c3 = __fadd_rn(p[3], p[7]);
    const float sum = __fadd_rn(__fadd_rn(c0, c2), __fadd_rn(c1, c3));
    if (q == 0) {
        const float value = bf16_rne(sum);
        if (logits && row < vocab) T::store(logits + row, value);
        cand[local] = row < vocab ? argmax_key(value, (uint32_t)row) : 0ull;
    }
    if (partial_best == nullptr) return;
    __syncthreads();
    if (tid < 16) {  // slot layout of the W8A8 head's candidates: 16 keys per CTA
        unsigned long long best = 0;
        if (tid == 0) {
#pragma unroll 8
            for (int r = 0; r < kQuadRowsPerCta; ++r) best = max(best, cand[r]);
        }
        partial_best[(size_t)blockIdx.x * 16 + tid] = best;
    }
}

bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace

cudaError_t init_head_bf16() {
    cudaError_t e = cudaFuncSetAttribute(head_bf16_kernel<Bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(head_bf16_kernel<F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(head_bf16_quad_kernel<Bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(head_bf16_quad_kernel<F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    return e;
}

}  // namespace w8a8

using namespace w8a8;

#define REQUIRE(cond, code)         \
    do {                            \
        if (!(cond)) return (code); \
    } while (0)

extern "C" int qwen3_head_bf16(const void *x, int dtype, const uint16_t *w, int vocab, int hidden, void *logits, uint32_t *token,
                               float *value, void *stream) {
    REQUIRE(device_status_ptr(), W8A8_ERR_NOT_INITIALIZED);
    REQUIRE(x && w && vocab > 0 && hidden > 0 && (logits || token), W8A8_ERR_BAD_ARG);
    REQUIRE(dtype == W8A8_BF16 || dtype == W8A8_F32, W8A8_ERR_BAD_ARG);
    REQUIRE(aligned(w, 2) && hidden <= 24576, W8A8_ERR_ALIGNMENT);
    const bool quad = hidden % 32 == 0 && aligned(w, 16);  // four threads per row, 16-byte loads
    const int per_cta = quad ? kQuadRowsPerCta : kRowsPerCta;
    const int blocks = (vocab + per_cta - 1) / per_cta;
    REQUIRE(token == nullptr || blocks <= kArgmaxMaxBlocks, W8A8_ERR_UNSUPPORTED);
    unsigned long long *partial = token ? argmax_scratch() : nullptr;
    const size_t smem = (size_t)hidden * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (quad)
        e = dtype == W8A8_BF16 ? launch_kernel(head_bf16_quad_kernel<Bf16>, dim3(blocks), dim3(kThreads), smem, s, (const uint16_t *)x, w, hidden,
                                               vocab, (uint16_t *)logits, partial)
                               : launch_kernel(head_bf16_quad_kernel<F32>, dim3(blocks), dim3(kThreads), smem, s, (const float *)x, w, hidden,
                                               vocab, (float *)logits, partial);
    else
        e = dtype == W8A8_BF16 ? launch_kernel(head_bf16_kernel<Bf16>, dim3(blocks), dim3(kThreads), smem, s, (const uint16_t *)x, w, hidden,
                                               vocab, (uint16_t *)logits, partial)
                               : launch_kernel(head_bf16_kernel<F32>, dim3(blocks), dim3(kThreads), smem, s, (const float *)x, w, hidden,
                                               vocab, (float *)logits, partial);
    if (e != cudaSuccess) return fail_cuda(e, "head_bf16 launch");
    if (token) {
        e = launch_argmax_finish(partial, blocks, 1, token, value, s);
        if (e != cudaSuccess) return fail_cuda(e, "head_bf16 selection launch");
    }
    return W8A8_OK;
}
