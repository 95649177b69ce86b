// Dynamic per-token INT8 activation quantizers, standalone and fused with the
// preceding RMSNorm or SwiGLU (sm_100a).
//
// What the reference computes (crates/inferrous-qwen3/):
//   quantize            src/kernels.rs:415-452   m = max(1e-8, max|x|); s = m/127; q = rne(clamp(x/s))
//   quantize_with_max   src/kernels.rs:455-475   same with m supplied by the producer
//   norm_quantize       src/kernels.rs:479-576   y = bf16((x*rsqrt(mean(x^2)+eps))*gain); quantize(y)
//   swiglu              src/kernels.rs:2172-2190 act = bf16((g/(1+exp(-g)))*u) (+ absmax publish)
//   residual            src/kernels.rs:2163-2170 bf16(a+b)
//
// Design here: one CTA per token row (256 or 512 threads; 1024 for a few rows), 128-bit global loads, the row kept
// in registers between the absmax pass and the coding pass (so it is read from HBM exactly once), warp-level
// redux for the absmax, a multiply with an exact-division fallback near rounding ties (quant_code,
// bit-identical to the reference's per-element division, no conversion-unit instructions), 4/8 int8 codes
// packed per store.  The sum of squares follows the reference's fixed tree (256 strided partials over a
// swizzled shared-memory copy of x, then distances 128..1) so that the bf16 norm row can match the reference
// bit for bit wherever rsqrt.approx does.  At thousands of rows these kernels are bound by instruction issue,
// not by HBM: requesting the next row ahead of time changed nothing, and the counters show two thirds of the
// cycles issuing with no pipe above 55 %.
#include "common.cuh"
#include "internal.h"

namespace w8a8 {
namespace {

constexpr int kThreads = 256;

struct QuantDev {
    const void *x;
    const void *x2;
    int64_t ld;
    int M, K;
    float eps;
    const uint32_t *maxima_in;
    int8_t *q;
    float *scale;
    void *y_out;
    uint32_t *maxima_reset;
    PrefetchHint hint;  // CTAs beyond the M row CTAs issue these L2 prefetches and leave
};

// Register-resident fast path: each thread keeps its RV 16-byte vectors of the row in registers between the
// absmax pass and the coding pass, so shared memory carries only the reductions (plain / SwiGLU) or the one
// copy of x that the reference's summation tree walks with stride 256 (RMSNorm; stored with a 16-byte XOR
// swizzle so that both the vector stores and the strided reads are bank-conflict free).
// Used whenever K <= RV * blockDim.x * kVec; the generic kernel below covers the rest.
template <class T, int MODE, int RV, int THREADS>
__global__ void __launch_bounds__(THREADS) quantize_rows_reg_kernel(const QuantDev a) {
    typedef typename T::storage S;
    constexpr int V = T::kVec;
    extern __shared__ __align__(16) float smem[];
    float *red = smem;                                           // 256 floats
    uint32_t *slots = reinterpret_cast<uint32_t *>(red + 256);  // 32 words
    float *row = smem + 256 + 32;                                // K floats, RMSNorm only
    const int tid = threadIdx.x;
    const int K = a.K;
    // float index swizzle: 16-byte group ^= bit 5 of the element index
    auto swz = [](int e) { return e ^ (((e >> 5) & 1) << 2); };

    if ((int)blockIdx.x >= a.M) {  // prefetch CTA: immutable weights only, so no dependency wait
        prefetch_ranges(a.hint, blockIdx.x - a.M, gridDim.x - a.M);
        return;
    }
    // Few rows (the 1024-thread shape): the gain row is a weight, so it is fetched before the dependency wait and
    // kept packed; the pass that needs it then waits on registers, not on L2.
    constexpr bool kEarlyGain = MODE == QUANT_RMSNORM && THREADS == 1024 && V == 8;  // (the f32 carrier would spill)
    uint4 gain_raw[kEarlyGain ? RV : 1];
    if (kEarlyGain) {
#pragma unroll
        for (int c = 0; c < RV; ++c) {
            const int j = (c * THREADS + tid) * V;
            if (j < K) gain_raw[c] = *reinterpret_cast<const uint4 *>(static_cast<const S *>(a.x2) + j);
        }
    }
    dependency_wait();

    for (int r = blockIdx.x; r < a.M; r += gridDim.x) {
        const S *xr = static_cast<const S *>(a.x) + (int64_t)r * a.ld;
        int8_t *qr = a.q + (int64_t)r * K;
        float v[RV][V];
        float m = 1e-8f;
#pragma unroll
        for (int c = 0; c < RV; ++c) {
            const int j = (c * THREADS + tid) * V;
            if (j < K) {
                Vec<T>::load(xr + j, v[c]);
                if (MODE == QUANT_SWIGLU) {
                    const S *ur = static_cast<const S *>(a.x2) + (int64_t)r * a.ld;
                    float u[V];
                    Vec<T>::load(ur + j, u);
#pragma unroll
                    for (int i = 0; i < V; ++i) v[c][i] = swiglu_value(v[c][i], u[i]);
                    if (a.y_out) Vec<T>::store(static_cast<S *>(a.y_out) + (int64_t)r * K + j, v[c]);
                }
                if (MODE == QUANT_RMSNORM) {
#pragma unroll
                    for (int i = 0; i < V; i += 4)
                        *reinterpret_cast<float4 *>(row + swz(j + i)) = make_float4(v[c][i], v[c][i + 1], v[c][i + 2], v[c][i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) m = fmaxf(m, fabsf(v[c][i]));  // fmaxf drops a NaN operand
                }
            }
        }
        if (MODE == QUANT_RMSNORM) {
            __syncthreads();
            if (tid < 256) {  // 256 strided partial sums, each added in index order (src/kernels.rs:508-519)
                float s = 0.0f;
                constexpr int kFull = RV * THREADS * V;  // the widest row of this instance
                if (K == kFull) {
                    // all loads first, then the chain of additions: swz(tid + 256 i) = swz(tid) + 256 i
                    const float *mine = row + swz(tid);
                    float x[kFull / 256];
#pragma unroll
                    for (int i = 0; i < kFull / 256; ++i) x[i] = mine[256 * i];
#pragma unroll
                    for (int i = 0; i < kFull / 256; ++i) s = __fadd_rn(s, __fmul_rn(x[i], x[i]));
                } else {
                    for (int j = tid; j < K; j += 256) {
                        const float x = row[swz(j)];
                        s = __fadd_rn(s, __fmul_rn(x, x));
                    }
                }
                red[tid] = s;
            }
            __syncthreads();
            if (tid < 32) {  // distances 128, 64, 32 then the warp distances 16..1 (src/kernels.rs:521-545)
                float t = __fadd_rn(__fadd_rn(__fadd_rn(red[tid], red[tid + 128]), __fadd_rn(red[tid + 64], red[tid + 192])),
                                    __fadd_rn(__fadd_rn(red[tid + 32], red[tid + 160]), __fadd_rn(red[tid + 96], red[tid + 224])));
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, d));
                if (tid == 0) red[0] = t;
            }
            __syncthreads();
            const float inv = rsqrt_approx(__fadd_rn(__fdiv_rn(red[0], (float)K), a.eps));
            const S *gr = static_cast<const S *>(a.x2);
#pragma unroll
            for (int c = 0; c < RV; ++c) {
                const int j = (c * THREADS + tid) * V;
                if (j < K) {
                    float g[V];
                    if (kEarlyGain)
                        Vec<T>::unpack(gain_raw[c], g);
                    else
                        Vec<T>::load(gr + j, g);
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        v[c][i] = bf16_rne(__fmul_rn(__fmul_rn(v[c][i], inv), g[i]));
                        m = fmaxf(m, fabsf(v[c][i]));
                    }
                    if (a.y_out) Vec<T>::store(static_cast<S *>(a.y_out) + (int64_t)r * K + j, v[c]);
                }
            }
        }
        const float s = __fdiv_rn(block_max(m, slots, tid), 127.0f);
        const float inv_s = __frcp_rn(s);
        if (tid == 0) {
            a.scale[r] = s;
            if (a.maxima_reset) a.maxima_reset[r] = __float_as_uint(1e-8f);
        }
#pragma unroll
        for (int c = 0; c < RV; ++c) {
            const int j = (c * THREADS + tid) * V;
            if (j < K) {
                int code[V];
#pragma unroll
                for (int i = 0; i < V; ++i) code[i] = quant_code(v[c][i], s, inv_s);
                store_codes<V>(qr + j, code);
            }
        }
        // block_max ends with a barrier, so red[] / slots[] / row[] are free for the next row
    }
}

// Launched with 256 threads per row, or 1024 when there are only a few rows (decode): the work per
// thread then shrinks to one or two 16-byte vectors and the kernel is one memory round trip long.
template <class T, int MODE>
__global__ void __launch_bounds__(1024) quantize_rows_kernel(const QuantDev a) {
    typedef typename T::storage S;
    constexpr int V = T::kVec;
    extern __shared__ __align__(16) float smem[];
    float *row = smem;                 // K floats
    float *red = smem + a.K;           // 256 floats
    uint32_t *slots = reinterpret_cast<uint32_t *>(red + 256);  // 32 words
    const int tid = threadIdx.x;
    const int K = a.K;
    const int nthreads = blockDim.x;

    if ((int)blockIdx.x >= a.M) {  // prefetch CTA: immutable weights only, so no dependency wait
        prefetch_ranges(a.hint, blockIdx.x - a.M, gridDim.x - a.M);
        return;
    }
    dependency_wait();

    for (int r = blockIdx.x; r < a.M; r += gridDim.x) {
        const S *xr = static_cast<const S *>(a.x) + (int64_t)r * a.ld;
        int8_t *qr = a.q + (int64_t)r * K;

        if (MODE == QUANT_WITH_MAX) {
            const float s = __fdiv_rn(__uint_as_float(a.maxima_in[r]), 127.0f);
            const float inv = __frcp_rn(s);
            if (tid == 0) a.scale[r] = s;
            for (int j = tid * V; j < K; j += nthreads * V) {
                float v[V];
                Vec<T>::load(xr + j, v);
                int c[V];
#pragma unroll
                for (int i = 0; i < V; ++i) c[i] = quant_code(v[i], s, inv);
                store_codes<V>(qr + j, c);
            }
            continue;
        }

        float m = 1e-8f;
        // pass 1: HBM -> registers -> shared (and the element-wise producer, if fused)
        for (int j = tid * V; j < K; j += nthreads * V) {
            float v[V];
            Vec<T>::load(xr + j, v);
            if (MODE == QUANT_SWIGLU) {
                const S *ur = static_cast<const S *>(a.x2) + (int64_t)r * a.ld;
                float u[V];
                Vec<T>::load(ur + j, u);
#pragma unroll
                for (int i = 0; i < V; ++i) v[i] = swiglu_value(v[i], u[i]);
                if (a.y_out) Vec<T>::store(static_cast<S *>(a.y_out) + (int64_t)r * K + j, v);
            }
            if (MODE != QUANT_RMSNORM) {
#pragma unroll
                for (int i = 0; i < V; ++i) m = fmaxf(m, fabsf(v[i]));  // fmaxf drops a NaN operand
            }
#pragma unroll
            for (int i = 0; i < V; i += 4)
                *reinterpret_cast<float4 *>(row + j + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }

        if (MODE == QUANT_RMSNORM) {
            __syncthreads();
            // 256 strided partial sums, each added in index order (src/kernels.rs:508-519)
            if (tid < 256) {
                float s = 0.0f;
                for (int j = tid; j < K; j += 256) s = __fadd_rn(s, __fmul_rn(row[j], row[j]));
                red[tid] = s;
            }
            __syncthreads();
            if (tid < 32) {
                // distances 128, 64, 32 then the warp distances 16..1 (src/kernels.rs:521-545)
                float t = __fadd_rn(__fadd_rn(__fadd_rn(red[tid], red[tid + 128]), __fadd_rn(red[tid + 64], red[tid + 192])),
                                    __fadd_rn(__fadd_rn(red[tid + 32], red[tid + 160]), __fadd_rn(red[tid + 96], red[tid + 224])));
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, d));
                if (tid == 0) red[0] = t;
            }
            __syncthreads();
            const float inv = rsqrt_approx(__fadd_rn(__fdiv_rn(red[0], (float)K), a.eps));
            const S *gr = static_cast<const S *>(a.x2);
            for (int j = tid * V; j < K; j += nthreads * V) {
                float g[V], y[V];
                Vec<T>::load(gr + j, g);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    y[i] = bf16_rne(__fmul_rn(__fmul_rn(row[j + i], inv), g[i]));
                    m = fmaxf(m, fabsf(y[i]));
                    row[j + i] = y[i];
                }
                if (a.y_out) Vec<T>::store(static_cast<S *>(a.y_out) + (int64_t)r * K + j, y);
            }
        }

        const float s = __fdiv_rn(block_max(m, slots, tid), 127.0f);
        const float inv = __frcp_rn(s);
        if (tid == 0) {
            a.scale[r] = s;
            if (a.maxima_reset) a.maxima_reset[r] = __float_as_uint(1e-8f);
        }
        // last pass: each thread re-reads exactly the elements it parked
        for (int j = tid * V; j < K; j += nthreads * V) {
            int c[V];
#pragma unroll
            for (int i = 0; i < V; ++i) c[i] = quant_code(row[j + i], s, inv);
            store_codes<V>(qr + j, c);
        }
        __syncthreads();  // row[] and red[] are reused by the next row of this CTA
    }
}

template <class T>
__global__ void __launch_bounds__(kThreads) swiglu_kernel(const typename T::storage *gate, const typename T::storage *up,
                                                          int I, int64_t ld, typename T::storage *act, uint32_t *maxima) {
    constexpr int V = T::kVec;
    __shared__ uint32_t slots[8];
    dependency_wait();
    const int r = blockIdx.y;
    const int j = (blockIdx.x * kThreads + threadIdx.x) * V;
    uint32_t key = 0;
    if (j < I) {
        float g[V], u[V];
        Vec<T>::load(gate + (int64_t)r * ld + j, g);
        Vec<T>::load(up + (int64_t)r * ld + j, u);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            g[i] = swiglu_value(g[i], u[i]);
            key = max(key, absmax_key(g[i]));
        }
        Vec<T>::store(act + (int64_t)r * I + j, g);
    }
    if (maxima) {
        key = warp_max_u32(key);
        if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = key;
        __syncthreads();
        if (threadIdx.x < 32) {
            key = warp_max_u32(slots[threadIdx.x & 7]);
            if (threadIdx.x == 0) atomicMax(maxima + r, key);
        }
    }
}

// Any row width and stride (no vector alignment assumed): one element per thread.
template <class T>
__global__ void __launch_bounds__(kThreads) swiglu_scalar_kernel(const typename T::storage *gate, const typename T::storage *up,
                                                                 int I, int64_t ld, typename T::storage *act, uint32_t *maxima) {
    __shared__ uint32_t slots[8];
    dependency_wait();
    const int r = blockIdx.y;
    const int j = blockIdx.x * kThreads + threadIdx.x;
    uint32_t key = 0;
    if (j < I) {
        const float v = swiglu_value(T::load(gate + (int64_t)r * ld + j), T::load(up + (int64_t)r * ld + j));
        key = absmax_key(v);
        T::store(act + (int64_t)r * I + j, v);
    }
    if (maxima) {
        key = warp_max_u32(key);
        if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = key;
        __syncthreads();
        if (threadIdx.x < 32) {
            key = warp_max_u32(slots[threadIdx.x & 7]);
            if (threadIdx.x == 0) atomicMax(maxima + r, key);
        }
    }
}

template <class T>
__global__ void __launch_bounds__(kThreads) residual_kernel(const typename T::storage *a, const typename T::storage *b,
                                                            size_t n, typename T::storage *out) {
    constexpr int V = T::kVec;
    dependency_wait();
    size_t i = ((size_t)blockIdx.x * kThreads + threadIdx.x) * V;
    if (i + V <= n) {
        float x[V], y[V];
        Vec<T>::load(a + i, x);
        Vec<T>::load(b + i, y);
#pragma unroll
        for (int k = 0; k < V; ++k) x[k] = bf16_rne(__fadd_rn(x[k], y[k]));
        Vec<T>::store(out + i, x);
    } else {
        for (; i < n; ++i) T::store(out + i, bf16_rne(__fadd_rn(T::load(a + i), T::load(b + i))));
    }
}

__global__ void rounding_probe_kernel(const float *x, int8_t *out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (int8_t)round_i8(x[i]);
}

constexpr int kMaxQuantSmem = 100 * 1024;
inline size_t quant_smem(int K) { return (size_t)(K + 256 + 32) * sizeof(float); }

template <class T, int MODE> cudaError_t launch_q(const QuantDev &d, cudaStream_t s) {
    // one CTA per row; with pending prefetch hints (few rows only) one more CTA per SM
    const int grid = d.M + (d.hint.count ? sm_count() : 0);
    if (MODE != QUANT_WITH_MAX) {
        // Register-resident kernels.  Few rows: 1024 threads so that the kernel is one memory round trip long.
        // Many rows: the smallest CTA that holds the row in <= 3 vectors per thread, which keeps the register
        // count low enough for 32-64 resident warps per SM (the bytes in flight that HBM needs).
        const size_t smem = (256 + 32 + (MODE == QUANT_RMSNORM ? (size_t)d.K : 0)) * sizeof(float);
        const int V = T::kVec;
        if (d.M > 64 && d.K <= 2 * 256 * V)
            return launch_kernel(quantize_rows_reg_kernel<T, MODE, 2, 256>, dim3(grid), dim3(256), smem, s, d);
        if (d.M > 64 && d.K <= 3 * 512 * V)
            return launch_kernel(quantize_rows_reg_kernel<T, MODE, 3, 512>, dim3(grid), dim3(512), smem, s, d);
        if (d.K <= 3 * 1024 * V)
            return launch_kernel(quantize_rows_reg_kernel<T, MODE, 3, 1024>, dim3(grid), dim3(1024), smem, s, d);
    }
    const int threads = d.M <= 64 ? 1024 : kThreads;  // few rows: one memory round trip per thread
    return launch_kernel(quantize_rows_kernel<T, MODE>, dim3(grid), dim3(threads), quant_smem(d.K), s, d);
}
template <class T, int MODE> cudaError_t set_attr() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(quantize_rows_kernel<T, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxQuantSmem))) return e;
    if (MODE != QUANT_WITH_MAX) {
        if ((e = cudaFuncSetAttribute(quantize_rows_reg_kernel<T, MODE, 3, 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxQuantSmem))) return e;
        if ((e = cudaFuncSetAttribute(quantize_rows_reg_kernel<T, MODE, 2, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxQuantSmem))) return e;
        if ((e = cudaFuncSetAttribute(quantize_rows_reg_kernel<T, MODE, 3, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxQuantSmem))) return e;
    }
    return cudaSuccess;
}

}  // namespace

cudaError_t init_quantize() {
    cudaError_t e;
#define W8A8_SET(T)                                                   \
    if ((e = set_attr<T, QUANT_PLAIN>()) != cudaSuccess) return e;    \
    if ((e = set_attr<T, QUANT_WITH_MAX>()) != cudaSuccess) return e; \
    if ((e = set_attr<T, QUANT_RMSNORM>()) != cudaSuccess) return e;  \
    if ((e = set_attr<T, QUANT_SWIGLU>()) != cudaSuccess) return e;
    W8A8_SET(Bf16)
    W8A8_SET(F32)
#undef W8A8_SET
    return cudaSuccess;
}

cudaError_t launch_quantize(const QuantArgs &a, cudaStream_t s) {
    if (quant_smem(a.K) > (size_t)kMaxQuantSmem) return cudaErrorInvalidValue;
    QuantDev d{a.x, a.x2, a.ld, a.M, a.K, a.eps, a.maxima_in, a.q, a.scale, a.y_out, a.maxima_reset, PrefetchHint{}};
    if (a.M <= kPrefetchMaxRows) d.hint = take_prefetch_hint();
#define W8A8_DISPATCH(T)                                                           \
    switch (a.mode) {                                                              \
        case QUANT_PLAIN: return launch_q<T, QUANT_PLAIN>(d, s);                   \
        case QUANT_WITH_MAX: return launch_q<T, QUANT_WITH_MAX>(d, s);             \
        case QUANT_RMSNORM: return launch_q<T, QUANT_RMSNORM>(d, s);               \
        case QUANT_SWIGLU: return launch_q<T, QUANT_SWIGLU>(d, s);                 \
        default: return cudaErrorInvalidValue;                                     \
    }
    if (a.dtype == 0) { W8A8_DISPATCH(Bf16) }
    W8A8_DISPATCH(F32)
#undef W8A8_DISPATCH
}

cudaError_t launch_swiglu(const void *gate, const void *up, int dtype, int M, int I, int64_t ld, void *act,
                          uint32_t *maxima, cudaStream_t s) {
    const int vec = dtype == 0 ? 8 : 4;
    const bool aligned = (I % vec == 0) && (ld % vec == 0) && ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                                                                 reinterpret_cast<uintptr_t>(act)) & 15u) == 0;
    if (!aligned) {
        dim3 grid((I + kThreads - 1) / kThreads, M);
        if (dtype == 0)
            swiglu_scalar_kernel<Bf16><<<grid, kThreads, 0, s>>>((const uint16_t *)gate, (const uint16_t *)up, I, ld, (uint16_t *)act, maxima);
        else
            swiglu_scalar_kernel<F32><<<grid, kThreads, 0, s>>>((const float *)gate, (const float *)up, I, ld, (float *)act, maxima);
        return cudaGetLastError();
    }
    if (dtype == 0) {
        dim3 grid((I + kThreads * 8 - 1) / (kThreads * 8), M);
        return launch_kernel(swiglu_kernel<Bf16>, grid, dim3(kThreads), (size_t)0, s, (const uint16_t *)gate, (const uint16_t *)up, I, ld, (uint16_t *)act, maxima);
    } else {
        dim3 grid((I + kThreads * 4 - 1) / (kThreads * 4), M);
        return launch_kernel(swiglu_kernel<F32>, grid, dim3(kThreads), (size_t)0, s, (const float *)gate, (const float *)up, I, ld, (float *)act, maxima);
    }
    return cudaGetLastError();
}

cudaError_t launch_residual(const void *a, const void *b, int dtype, size_t n, void *out, cudaStream_t s) {
    if (dtype == 0) {
        size_t blocks = (n + kThreads * 8 - 1) / (kThreads * 8);
        return launch_kernel(residual_kernel<Bf16>, dim3((unsigned)blocks), dim3(kThreads), (size_t)0, s, (const uint16_t *)a, (const uint16_t *)b, n, (uint16_t *)out);
    } else {
        size_t blocks = (n + kThreads * 4 - 1) / (kThreads * 4);
        return launch_kernel(residual_kernel<F32>, dim3((unsigned)blocks), dim3(kThreads), (size_t)0, s, (const float *)a, (const float *)b, n, (float *)out);
    }
    return cudaGetLastError();
}

cudaError_t launch_rounding_probe(const float *x, int8_t *out, size_t n, cudaStream_t s) {
    rounding_probe_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, out, n);
    return cudaGetLastError();
}

}  // namespace w8a8
