// One-thread-per-output W8A8 projection: the on-GPU statement of the operator that every
// fast variant must equal bit for bit.  It plays the role the reference gives its own
// `linear` kernel (crates/inferrous-qwen3/src/kernels.rs:808-845), which its conformance
// tests use as the oracle for every other variant (src/conformance.rs:208-219).
#include "common.cuh"
#include "internal.h"

namespace w8a8 {
namespace {

struct NaiveDev {
    const int8_t *q;
    const float *a_scale;
    int M, K, count;
    const int8_t *w[kMaxGroup];
    const float *ws[kMaxGroup];
    void *out[kMaxGroup];
    int n[kMaxGroup];
    const void *residual;
    void *combined;
    void *act;
    uint32_t *maxima;
    int32_t *acc;
};

__device__ __forceinline__ int dot_row(const int8_t *a, const int8_t *b, int K) {
    int acc = 0;
    for (int k = 0; k < K; k += 4) {
        int x = *reinterpret_cast<const int *>(a + k);
        int y = *reinterpret_cast<const int *>(b + k);
        acc = __dp4a(x, y, acc);
    }
    return acc;
}

template <class T, int EPI>
__global__ void naive_linear_kernel(const NaiveDev a) {
    typedef typename T::storage S;
    dependency_wait();
    const int ntot = (EPI == EPI_SWIGLU) ? a.n[0] : a.n[0] + (a.count > 1 ? a.n[1] : 0) + (a.count > 2 ? a.n[2] : 0);
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)a.M * ntot) return;
    const int m = (int)(idx / ntot);
    int c = (int)(idx % ntot);
    const int8_t *qr = a.q + (int64_t)m * a.K;
    if (EPI == EPI_SWIGLU) {
        const float g = dequant(dot_row(qr, a.w[0] + (int64_t)c * a.K, a.K), a.a_scale[m], a.ws[0][c]);
        const float u = dequant(dot_row(qr, a.w[1] + (int64_t)c * a.K, a.K), a.a_scale[m], a.ws[1][c]);
        const float v = swiglu_value(g, u);
        const int64_t o = (int64_t)m * a.n[0] + c;
        if (a.out[0]) T::store(static_cast<S *>(a.out[0]) + o, g);
        if (a.out[1]) T::store(static_cast<S *>(a.out[1]) + o, u);
        T::store(static_cast<S *>(a.act) + o, v);
        if (a.maxima) atomicMax(a.maxima + m, absmax_key(v));
        return;
    }
    int g = 0;
    while (g + 1 < a.count && c >= a.n[g]) { c -= a.n[g]; ++g; }
    const int acc = dot_row(qr, a.w[g] + (int64_t)c * a.K, a.K);
    const int64_t o = (int64_t)m * a.n[g] + c;
    if (EPI == EPI_ACC) { a.acc[o] = acc; return; }
    const float y = dequant(acc, a.a_scale[m], a.ws[g][c]);
    if (a.out[g]) T::store(static_cast<S *>(a.out[g]) + o, y);
    if (EPI == EPI_RESIDUAL) {
        const float r = T::load(static_cast<const S *>(a.residual) + o);
        T::store(static_cast<S *>(a.combined) + o, bf16_rne(__fadd_rn(r, y)));
    }
}

template <class T> cudaError_t launch(const LinearArgs &l, const NaiveDev &d, cudaStream_t s) {
    int ntot = 0;
    for (int g = 0; g < l.count; ++g) ntot += l.n[g];
    if (l.epilogue == EPI_SWIGLU) ntot = l.n[0];
    const int64_t total = (int64_t)l.M * ntot;
    const unsigned blocks = (unsigned)((total + 127) / 128);
    switch (l.epilogue) {
        case EPI_PLAIN: naive_linear_kernel<T, EPI_PLAIN><<<blocks, 128, 0, s>>>(d); break;
        case EPI_RESIDUAL: naive_linear_kernel<T, EPI_RESIDUAL><<<blocks, 128, 0, s>>>(d); break;
        case EPI_SWIGLU: naive_linear_kernel<T, EPI_SWIGLU><<<blocks, 128, 0, s>>>(d); break;
        case EPI_ACC: naive_linear_kernel<T, EPI_ACC><<<blocks, 128, 0, s>>>(d); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_linear_naive(const LinearArgs &l, cudaStream_t s) {
    NaiveDev d{};
    d.q = l.q; d.a_scale = l.a_scale; d.M = l.M; d.K = l.K; d.count = l.count;
    for (int g = 0; g < kMaxGroup; ++g) { d.w[g] = l.w[g]; d.ws[g] = l.ws[g]; d.out[g] = l.out[g]; d.n[g] = l.n[g]; }
    d.residual = l.residual; d.combined = l.combined; d.act = l.act; d.maxima = l.maxima; d.acc = l.acc;
    return l.dtype == 0 ? launch<Bf16>(l, d, s) : launch<F32>(l, d, s);
}

}  // namespace w8a8
