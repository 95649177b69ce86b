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
// What differs is how the bytes move: a warp works on two rows at once with 16 two-byte loads per row in flight per lane
// (a warp-wide load covers 64 contiguous bytes; consecutive loads finish the 128-byte line), the activation row is
// parked in shared memory once per CTA, and the greedy selection is fused in: a CTA of 8 warps leaves the best
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

bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace

cudaError_t init_head_bf16() {
    cudaError_t e = cudaFuncSetAttribute(head_bf16_kernel<Bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    return e == cudaSuccess ? cudaFuncSetAttribute(head_bf16_kernel<F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) : e;
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
    const int blocks = (vocab + kRowsPerCta - 1) / kRowsPerCta;
    REQUIRE(token == nullptr || blocks <= kArgmaxMaxBlocks, W8A8_ERR_UNSUPPORTED);
    unsigned long long *partial = token ? argmax_scratch() : nullptr;
    const size_t smem = (size_t)hidden * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = dtype == W8A8_BF16
                        ? launch_kernel(head_bf16_kernel<Bf16>, dim3(blocks), dim3(kThreads), smem, s, (const uint16_t *)x, w, hidden, vocab,
                                        (uint16_t *)logits, partial)
                        : launch_kernel(head_bf16_kernel<F32>, dim3(blocks), dim3(kThreads), smem, s, (const float *)x, w, hidden, vocab,
                                        (float *)logits, partial);
    if (e != cudaSuccess) return fail_cuda(e, "head_bf16 launch");
    if (token) {
        e = launch_argmax_finish(partial, blocks, 1, token, value, s);
        if (e != cudaSuccess) return fail_cuda(e, "head_bf16 selection launch");
    }
    return W8A8_OK;
}
