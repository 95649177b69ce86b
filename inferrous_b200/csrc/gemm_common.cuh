// Shared by the tensor-core GEMM kernels: kernel parameters and the accumulator drain
// (tensor memory -> registers -> dequantize -> bf16 -> global), 32 columns at a time.
#pragma once
#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace w8a8 {

struct GemmDev {
    const float *a_scale;
    const float *w_scale;
    int M, N, K;
    void *y;
    const void *residual;
    void *combined;
    int32_t *acc;
    uint32_t *status;
};

// One thread finishes 32 consecutive output channels of its row m from raw accumulators:
// y[m, n0 + i] = bf16((f32(v[i]) * a_scale[m]) * w_scale[n0 + i]), optional residual sum, or the raw int32.
template <class T, int EPI>
__device__ __forceinline__ void emit_columns(const GemmDev &p, const int (&v)[32], int m, float as, int n0) {
    typedef typename T::storage S;
    const int64_t o = (int64_t)m * p.N + n0;
    const bool full = (n0 + 32 <= p.N);
    if (EPI == EPI_ACC) {
        if (full && (p.N & 3) == 0) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<int4 *>(p.acc + o + i) = make_int4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        } else {
            for (int i = 0; i < 32 && n0 + i < p.N; ++i) p.acc[o + i] = v[i];
        }
        return;
    }
    if (full && (p.N % T::kVec) == 0) {
#pragma unroll
        for (int i = 0; i < 32; i += T::kVec) {
            float y[T::kVec];
#pragma unroll
            for (int j = 0; j < T::kVec; j += 4) {
                const float4 w4 = __ldg(reinterpret_cast<const float4 *>(p.w_scale + n0 + i + j));
                y[j + 0] = dequant(v[i + j + 0], as, w4.x);
                y[j + 1] = dequant(v[i + j + 1], as, w4.y);
                y[j + 2] = dequant(v[i + j + 2], as, w4.z);
                y[j + 3] = dequant(v[i + j + 3], as, w4.w);
            }
            if (p.y) Vec<T>::store(static_cast<S *>(p.y) + o + i, y);
            if (EPI == EPI_RESIDUAL) {
                float r[T::kVec];
                Vec<T>::load(static_cast<const S *>(p.residual) + o + i, r);
#pragma unroll
                for (int j = 0; j < T::kVec; ++j) r[j] = bf16_rne(__fadd_rn(r[j], y[j]));
                Vec<T>::store(static_cast<S *>(p.combined) + o + i, r);
            }
        }
    } else {
        for (int i = 0; i < 32 && n0 + i < p.N; ++i) {
            const float y = dequant(v[i], as, p.w_scale[n0 + i]);
            if (p.y) T::store(static_cast<S *>(p.y) + o + i, y);
            if (EPI == EPI_RESIDUAL) {
                const float r = T::load(static_cast<const S *>(p.residual) + o + i);
                T::store(static_cast<S *>(p.combined) + o + i, bf16_rne(__fadd_rn(r, y)));
            }
        }
    }
}

// One thread drains `width` columns of its own accumulator row (TMEM lane) starting at t_row, 32 at a time.
// All 32 lanes of the warp must call it together (tcgen05.ld is warp-collective); rows beyond M only load.
template <class T, int EPI>
__device__ __forceinline__ void drain_accumulator(const GemmDev &p, uint32_t t_row, int m, bool m_ok, float as, int n_base,
                                                  int width) {
#pragma unroll 1
    for (int c = 0; c < width / 32; ++c) {
        const int n0 = n_base + c * 32;
        if (n0 >= p.N) break;  // warp-uniform
        int v[32];
        tmem_ld_32x32(t_row + (uint32_t)(c * 32), v);
        tmem_ld_wait();
        if (m_ok) emit_columns<T, EPI>(p, v, m, as, n0);
    }
}

}  // namespace w8a8
