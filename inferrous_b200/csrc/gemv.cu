// Decode-regime W8A8 projections (few tokens, HBM-bound): stream the int8 weights once with
// coalesced 16-byte loads and do the integer dot products on the fly (sm_100a).
//
// Replaces, from crates/inferrous-qwen3/src/kernels.rs:
//   linear (:808-845), scaled_dot (:270-291), linear_pair / linear_triple (:698-806),
//   linear_residual (:579-618), linear_swiglu (:621-695), linear_splitk (:935-1034).
// The reference gives each output channel to one warp that walks the row 4 bytes per lane.
// Here:
//   gemv_dp4a  (M <= 4)   one warp per output channel, 16 bytes per lane per load, up to eight
//                         loads in flight per lane, dp4a against activations parked in shared
//                         memory, optional split of K over the warps of a CTA (exact: int32).
//   gemv_mma   (M <= 64)  one CTA per 16 output channels; the eight warps split K; each lane
//                         streams 16-byte pieces of two weight rows straight into the A
//                         fragments of mma.sync.m16n8k32.s8 (K is consumed in a permuted order,
//                         which integer accumulation allows), tokens are the MMA's N side.
// Weight loads are issued before griddepcontrol.wait: weights are immutable, only the
// activations depend on the preceding kernel.
#include "common.cuh"
#include "internal.h"

namespace w8a8 {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

struct GemvDev {
    const int8_t *q;
    const float *a_scale;
    int M, K, count;
    const int8_t *w[kMaxGroup];
    const float *ws[kMaxGroup];
    void *out[kMaxGroup];
    int n[kMaxGroup];
    int ntot;  // rows to iterate: sum of n[], or n[0] for the fused gate/up epilogue
    int ks;    // warps that share one output channel (dp4a kernel): 1, 2, 4 or 8
    const void *residual;
    void *combined;
    void *act;
    uint32_t *maxima;
    int32_t *acc;
    unsigned long long *partial_best;
    // quantizing prologue (SRC != SRC_CODES)
    const void *x;
    const void *gamma;
    float eps;
    const uint32_t *maxima_in;
    uint32_t *maxima_reset;
    int reset_words;
    int8_t *q_out;
    float *scale_out;
    PushTarget push;
};

// One 8-byte packet {value bits, tag of the call} to the same slot of every rank (plain peer stores over NVLink).
__device__ __forceinline__ void push_packet(const PushTarget &t, uint32_t call, size_t element, float value) {
    const size_t at = ((size_t)(call & 1u) * t.tp + t.rank) * t.slot + element;
    const uint32_t bits = __float_as_uint(value), tag = call + 1u;
    for (int p = 0; p < t.tp; ++p)
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(t.ll[p] + at), "r"(bits), "r"(tag) : "memory");
}

__device__ __forceinline__ int dp4a_16(const uint4 &w, const uint4 &a, int acc) {
    acc = __dp4a((int)w.x, (int)a.x, acc);
    acc = __dp4a((int)w.y, (int)a.y, acc);
    acc = __dp4a((int)w.z, (int)a.z, acc);
    acc = __dp4a((int)w.w, (int)a.w, acc);
    return acc;
}

// Which matrix of the group a global row index falls in.
__device__ __forceinline__ void locate(const GemvDev &a, int row, int &g, int &c) {
    g = 0;
    c = row;
    if (a.count > 1 && c >= a.n[0]) {
        c -= a.n[0];
        g = 1;
        if (a.count > 2 && c >= a.n[1]) {
            c -= a.n[1];
            g = 2;
        }
    }
}

// The activation quantizer as a prologue of the one-token GEMV: every CTA turns the unquantized row into int8 codes
// in its own shared memory while its first weight loads are in flight, so that no quantizer kernel (and no launch
// gap) sits between the producer of the row and the projection.  The arithmetic is that of the standalone
// quantizers (quantize.cu), pass for pass:
//   SRC_WITH_MAX  quantize_with_max (src/kernels.rs:455-475): s = m / 127 with m published by the producer
//   SRC_RMSNORM   norm_quantize (src/kernels.rs:479-576): the reference's summation tree (256 strided partial sums,
//                 distances 128..1), y = bf16((x * rsqrt(mean + eps)) * gain), m = max(1e-8, max|y|), s = m / 127
// `extra` is K + 256 + 32 floats of shared memory for SRC_RMSNORM (unused for SRC_WITH_MAX).  Returns the scale.
template <class T, int SRC>
__device__ __forceinline__ float quantize_prologue(const GemvDev &a, int8_t *sq, float *extra, int tid) {
    typedef typename T::storage S;
    constexpr int V = T::kVec;
    const int K = a.K;
    const S *xr = static_cast<const S *>(a.x);
    float s;
    if constexpr (SRC == SRC_WITH_MAX) {
        s = __fdiv_rn(__uint_as_float(a.maxima_in[0]), 127.0f);
        const float inv = __frcp_rn(s);
        for (int j = tid * V; j < K; j += kThreads * V) {
            float v[V];
            Vec<T>::load(xr + j, v);
            int c[V];
#pragma unroll
            for (int i = 0; i < V; ++i) c[i] = quant_code(v[i], s, inv);
            store_codes<V>(sq + j, c);
        }
    } else {
        float *row = extra;
        float *red = extra + K;
        uint32_t *slots = reinterpret_cast<uint32_t *>(red + 256);
        for (int j = tid * V; j < K; j += kThreads * V) {
            float v[V];
            Vec<T>::load(xr + j, v);
#pragma unroll
            for (int i = 0; i < V; i += 4)
                *reinterpret_cast<float4 *>(row + j + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
        __syncthreads();
        {
            float p = 0.0f;
            for (int j = tid; j < K; j += 256) p = __fadd_rn(p, __fmul_rn(row[j], row[j]));
            red[tid] = p;
        }
        __syncthreads();
        if (tid < 32) {
            float t = __fadd_rn(__fadd_rn(__fadd_rn(red[tid], red[tid + 128]), __fadd_rn(red[tid + 64], red[tid + 192])),
                                __fadd_rn(__fadd_rn(red[tid + 32], red[tid + 160]), __fadd_rn(red[tid + 96], red[tid + 224])));
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, d));
            if (tid == 0) red[0] = t;
        }
        __syncthreads();
        const float inv_norm = rsqrt_approx(__fadd_rn(__fdiv_rn(red[0], (float)K), a.eps));
        const S *gr = static_cast<const S *>(a.gamma);
        float m = 1e-8f;
        for (int j = tid * V; j < K; j += kThreads * V) {
            float g[V];
            Vec<T>::load(gr + j, g);
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const float y = bf16_rne(__fmul_rn(__fmul_rn(row[j + i], inv_norm), g[i]));
                m = fmaxf(m, fabsf(y));
                row[j + i] = y;
            }
        }
        s = __fdiv_rn(block_max(m, slots, tid), 127.0f);
        const float inv = __frcp_rn(s);
        for (int j = tid * V; j < K; j += kThreads * V) {
            int c[V];
#pragma unroll
            for (int i = 0; i < V; ++i) c[i] = quant_code(row[j + i], s, inv);
            store_codes<V>(sq + j, c);
        }
    }
    if (blockIdx.x == 0 && tid == 0) {
        if (a.scale_out) a.scale_out[0] = s;
        for (int i = 0; i < a.reset_words; ++i) a.maxima_reset[i] = __float_as_uint(1e-8f);
    }
    return s;
}

// ---------------------------------------------------------------------------------------
// gemv_dp4a: MT tokens (1..4), R = 1 (plain) or 2 (gate+up) weight rows per warp.
// SRC != SRC_CODES (MT == 1 only): the activation row is quantized in the prologue.
// ---------------------------------------------------------------------------------------
template <int MT, class T, int EPI, int SRC = SRC_CODES>
__global__ void __launch_bounds__(kThreads) gemv_dp4a_kernel(const GemvDev a) {
    typedef typename T::storage S;
    constexpr int R = (EPI == EPI_SWIGLU) ? 2 : 1;
    constexpr int U = (EPI == EPI_SWIGLU) ? 4 : 8;  // 16-byte loads in flight per lane per row
    extern __shared__ __align__(16) uint8_t smem_raw[];
    int8_t *sq = reinterpret_cast<int8_t *>(smem_raw);                         // [MT][K]
    int *red = reinterpret_cast<int *>(smem_raw + (size_t)MT * a.K);           // [kWarps][R*MT]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = a.K, KS = a.ks;
    const int rows_per_cta = kWarps / KS;
    const int row = blockIdx.x * rows_per_cta + warp / KS;  // global row of this warp
    const int kslot = warp % KS;
    const bool live = row < a.ntot;

    int g = 0, c = 0;
    const int8_t *wr[R];
    if (live) {
        if (EPI == EPI_SWIGLU) {
            c = row;
            wr[0] = a.w[0] + (int64_t)c * K;
            wr[R - 1] = a.w[1] + (int64_t)c * K;
        } else {
            locate(a, row, g, c);
            wr[0] = a.w[g] + (int64_t)c * K;
        }
    }

    int acc[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0;

    const int step = KS * 512;                // bytes of K between this warp's consecutive chunks
    const int first = kslot * 512 + lane * 16;

    // First batch of weight loads goes out before anything that depends on the predecessor.
    uint4 wv[R][U];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int off = first + u * step;
            wv[r][u] = (live && off < K) ? ld_stream_16(wr[r] + off) : make_uint4(0, 0, 0, 0);
        }

    // What the epilogue needs is fetched early, so that the end of the kernel waits on registers only: the channel's
    // weight scale(s) now (immutable), the token's activation scale and residual element right after the dependency
    // wait.  Lane m of the warp finishes token m.
    float ws_pre[R];
#pragma unroll
    for (int r = 0; r < R; ++r) ws_pre[r] = 0.0f;
    if (live && EPI != EPI_ACC) {
        if (EPI == EPI_SWIGLU) {
            ws_pre[0] = a.ws[0][c];
            ws_pre[R - 1] = a.ws[1][c];
        } else {
            ws_pre[0] = a.ws[g][c];
        }
    }

    dependency_wait();
    float as_pre = 0.0f, res_pre = 0.0f;
    uint32_t call_pre = 0;
    if (EPI == EPI_PUSH) call_pre = *reinterpret_cast<const volatile uint32_t *>(a.push.seq);
    if (live && lane < MT) {
        if (EPI != EPI_ACC && SRC == SRC_CODES) as_pre = a.a_scale[lane];
        if (EPI == EPI_RESIDUAL) res_pre = T::load(static_cast<const S *>(a.residual) + (int64_t)lane * a.n[g] + c);
    }
    float own_scale = 0.0f;
    if constexpr (SRC == SRC_CODES) {
        // Park the quantized activations (MT rows of K bytes) in shared memory.
        for (int i = tid * 16; i < MT * K; i += kThreads * 16)
            *reinterpret_cast<uint4 *>(sq + i) = *reinterpret_cast<const uint4 *>(a.q + i);
    } else {
        static_assert(SRC == SRC_CODES || MT == 1, "the quantizing prologue handles one token");
        own_scale = quantize_prologue<T, SRC>(a, sq, reinterpret_cast<float *>(red + kWarps * 2 * MT), tid);
    }
    __syncthreads();
    if constexpr (SRC != SRC_CODES) {
        if (blockIdx.x == 0 && a.q_out)
            for (int i = tid * 16; i < K; i += kThreads * 16)
                *reinterpret_cast<uint4 *>(a.q_out + i) = *reinterpret_cast<const uint4 *>(sq + i);
    }

    for (int base = first; base < K; base += U * step) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int off = base + u * step;
            if (off < K) {
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const uint4 av = *reinterpret_cast<const uint4 *>(sq + m * K + off);
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[r][m] = dp4a_16(wv[r][u], av, acc[r][m]);
                }
            }
        }
        const int next = base + U * step;
        if (next - lane * 16 < K) {  // warp-uniform: does any lane still have bytes to fetch
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int off = next + u * step;
                    wv[r][u] = (live && off < K) ? ld_stream_16(wr[r] + off) : make_uint4(0, 0, 0, 0);
                }
        }
    }

#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = warp_sum_i32(acc[r][m]);

    if (KS > 1) {  // exact int32 reduction over the warps that split K
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) red[warp * (R * MT) + r * MT + m] = acc[r][m];
        }
        __syncthreads();
        if (kslot != 0) return;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                int s = 0;
                for (int k = 0; k < KS; ++k) s += red[(warp + k) * (R * MT) + r * MT + m];
                acc[r][m] = s;
            }
    }
    if (!live || lane >= MT) return;

    // lane m finishes token m
    int sum[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        sum[r] = acc[r][0];
#pragma unroll
        for (int m = 1; m < MT; ++m)
            if (lane == m) sum[r] = acc[r][m];
    }
    const int m = lane;
    const float as = (SRC == SRC_CODES) ? as_pre : own_scale;
    if (EPI == EPI_ACC) {
        a.acc[(int64_t)m * a.n[0] + c] = sum[0];
    } else if (EPI == EPI_SWIGLU) {
        const float gv = dequant(sum[0], as, ws_pre[0]);
        const float uv = dequant(sum[R - 1], as, ws_pre[R - 1]);
        const float v = swiglu_value(gv, uv);
        const int64_t o = (int64_t)m * a.n[0] + c;
        if (a.out[0]) T::store(static_cast<S *>(a.out[0]) + o, gv);
        if (a.out[1]) T::store(static_cast<S *>(a.out[1]) + o, uv);
        T::store(static_cast<S *>(a.act) + o, v);
        if (a.maxima) atomicMax(a.maxima + m, absmax_key(v));
    } else if (EPI == EPI_PUSH) {
        push_packet(a.push, call_pre, (size_t)m * a.n[0] + c, dequant(sum[0], as, ws_pre[0]));
    } else {
        const float y = dequant(sum[0], as, ws_pre[0]);
        const int64_t o = (int64_t)m * a.n[g] + c;
        if (a.out[g]) T::store(static_cast<S *>(a.out[g]) + o, y);
        if (EPI == EPI_RESIDUAL) T::store(static_cast<S *>(a.combined) + o, bf16_rne(__fadd_rn(res_pre, y)));
    }
}

// ---------------------------------------------------------------------------------------
// gemv_mma: NT tiles of 8 tokens; one CTA per block of 16 output channels; warps split K.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, class T, int EPI>
__global__ void __launch_bounds__(kThreads) gemv_mma_kernel(const GemvDev a) {
    typedef typename T::storage S;
    __shared__ int red[kWarps][NT * 4 * 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t = lane & 3;
    const int K = a.K;

    // row block -> matrix of the group (blocks never straddle matrices: each matrix is padded
    // to whole 16-row blocks by the launcher's block count)
    int blk = blockIdx.x, g = 0;
    while (g + 1 < a.count && blk >= (a.n[g] + 15) / 16) { blk -= (a.n[g] + 15) / 16; ++g; }
    const int n = a.n[g];
    const int c0 = blk * 16;
    const int r_lo = min(c0 + gq, n - 1), r_hi = min(c0 + gq + 8, n - 1);  // clamped: extra rows are discarded
    const int8_t *w_lo = a.w[g] + (int64_t)r_lo * K + t * 16;
    const int8_t *w_hi = a.w[g] + (int64_t)r_hi * K + t * 16;

    int acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0;

    // This warp owns the 128-byte K steps s with s % kWarps == warp; two steps are in flight,
    // held in two explicitly named register buffers.
    const int nsteps = K / 128;
    uint4 lo0[2], hi0[2], lo1[2], hi1[2];
    auto load_w = [&](int s, uint4(&lo)[2], uint4(&hi)[2]) {
        if (s < nsteps) {
            const int k0 = s * 128;
            lo[0] = ld_stream_16(w_lo + k0);
            lo[1] = ld_stream_16(w_lo + k0 + 64);
            hi[0] = ld_stream_16(w_hi + k0);
            hi[1] = ld_stream_16(w_hi + k0 + 64);
        }
    };
    load_w(warp, lo0, hi0);
    load_w(warp + kWarps, lo1, hi1);

    dependency_wait();

    // Token fragments travel with the weights: they are fetched one step ahead of their use, so the MMAs of a
    // step wait on nothing but registers.
    const int8_t *qb = a.q + t * 16;
    uint4 b0[2][NT], b1[2][NT];
    auto load_b = [&](int s, uint4(&b)[2][NT]) {
        if (s < nsteps) {
            const int k0 = s * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int tok = j * 8 + gq;
                    b[h][j] = tok < a.M ? *reinterpret_cast<const uint4 *>(qb + (int64_t)tok * K + k0 + h * 64) : make_uint4(0, 0, 0, 0);
                }
        }
    };
    auto compute = [&](const uint4(&lo)[2], const uint4(&hi)[2], const uint4(&b)[2][NT]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 r = lo[h], v = hi[h];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 p = b[h][j];
                mma_s8(acc[j], r.x, v.x, r.y, v.y, p.x, p.y);
                mma_s8(acc[j], r.z, v.z, r.w, v.w, p.z, p.w);
            }
        }
    };
    load_b(warp, b0);
    load_b(warp + kWarps, b1);
    for (int s = warp; s < nsteps; s += 2 * kWarps) {
        compute(lo0, hi0, b0);
        load_w(s + 2 * kWarps, lo0, hi0);
        load_b(s + 2 * kWarps, b0);
        if (s + kWarps < nsteps) {
            compute(lo1, hi1, b1);
            load_w(s + 3 * kWarps, lo1, hi1);
            load_b(s + 3 * kWarps, b1);
        }
    }

#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][(j * 4 + i) * 32 + lane] = acc[j][i];
    __syncthreads();

    __shared__ unsigned long long cand[(EPI == EPI_ARGMAX) ? NT * 8 * 16 : 1];  // [token][row of the block]
    for (int idx = tid; idx < NT * 128; idx += kThreads) {
        int sum = 0;
#pragma unroll
        for (int k = 0; k < kWarps; ++k) sum += red[k][idx];
        const int l = idx & 31, reg = (idx >> 5) & 3, j = idx >> 7;
        const int row = c0 + (l >> 2) + 8 * (reg >> 1);
        const int tok = j * 8 + 2 * (l & 3) + (reg & 1);
        if (EPI == EPI_ARGMAX) {
            // the logit itself is never stored: only this block's best (value, index) per token survives
            unsigned long long key = 0;
            if (row < n && tok < a.M) key = argmax_key(dequant(sum, a.a_scale[tok], a.ws[g][row]), (uint32_t)row);
            cand[tok * 16 + (row - c0)] = key;
            continue;
        }
        if (row >= n || tok >= a.M) continue;
        const int64_t o = (int64_t)tok * n + row;
        if (EPI == EPI_ACC) {
            a.acc[o] = sum;
            continue;
        }
        if (EPI == EPI_PUSH) {
            push_packet(a.push, *reinterpret_cast<const volatile uint32_t *>(a.push.seq), (size_t)o,
                        dequant(sum, a.a_scale[tok], a.ws[g][row]));
            continue;
        }
        const float y = dequant(sum, a.a_scale[tok], a.ws[g][row]);
        if (a.out[g]) T::store(static_cast<S *>(a.out[g]) + o, y);
        if (EPI == EPI_RESIDUAL) {
            const float res = T::load(static_cast<const S *>(a.residual) + o);
            T::store(static_cast<S *>(a.combined) + o, bf16_rne(__fadd_rn(res, y)));
        }
    }
    if (EPI == EPI_ARGMAX) {
        __syncthreads();
        if (tid < 16) {  // thread = token: best of the block's 16 channels (16 candidates per block, absent tokens 0)
            unsigned long long best = 0;
            if (tid < NT * 8) {
#pragma unroll
                for (int r = 0; r < 16; ++r) best = max(best, cand[tid * 16 + r]);
            }
            a.partial_best[(size_t)blockIdx.x * 16 + tid] = best;
        }
    }
}

// Reduces the per-block candidates of the fused head projection to one token per row of activations:
// the largest finite logit, the lowest index among equals, ~0 when any logit of the row was not finite.
__global__ void __launch_bounds__(1024) argmax_finish_kernel(const unsigned long long *partial, int blocks, uint32_t *token,
                                                             float *value) {
    __shared__ unsigned long long slots[32];
    dependency_wait();
    const int m = blockIdx.x, t = threadIdx.x;
    unsigned long long best = 0;
    for (int b = t; b < blocks; b += 1024) best = max(best, partial[(size_t)b * 16 + m]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) best = max(best, __shfl_down_sync(0xffffffffu, best, d));
    if ((t & 31) == 0) slots[t >> 5] = best;
    __syncthreads();
    if (t < 32) {
        best = slots[t];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) best = max(best, __shfl_down_sync(0xffffffffu, best, d));
        if (t == 0) {
            const bool bad = best == ~0ull || best == 0ull;
            token[m] = bad ? 0xffffffffu : 0xffffffffu - (uint32_t)(best & 0xffffffffull);
            if (value) {
                const uint32_t o = (uint32_t)(best >> 32);
                const uint32_t bits = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
                value[m] = bad ? __uint_as_float(0x7fc00000u) : __uint_as_float(bits);
            }
        }
    }
}

GemvDev make_dev(const LinearArgs &l) {
    GemvDev d{};
    d.q = l.q; d.a_scale = l.a_scale; d.M = l.M; d.K = l.K; d.count = l.count;
    int ntot = 0;
    for (int g = 0; g < kMaxGroup; ++g) {
        d.w[g] = l.w[g]; d.ws[g] = l.ws[g]; d.out[g] = l.out[g]; d.n[g] = l.n[g];
        if (g < l.count) ntot += l.n[g];
    }
    d.ntot = (l.epilogue == EPI_SWIGLU) ? l.n[0] : ntot;
    d.ks = 1;
    d.residual = l.residual; d.combined = l.combined; d.act = l.act; d.maxima = l.maxima; d.acc = l.acc;
    d.partial_best = l.partial_best;
    d.x = l.x; d.gamma = l.gamma; d.eps = l.eps; d.maxima_in = l.maxima_in; d.maxima_reset = l.maxima_reset;
    d.reset_words = l.maxima_reset ? l.reset_words : 0; d.q_out = l.q_out; d.scale_out = l.scale_out;
    d.push = l.push;
    return d;
}

constexpr int kMaxDp4aSmem = 4 * 24576 + 1024;

template <int MT, class T, int EPI> cudaError_t launch_dp4a_inst(const GemvDev &d, cudaStream_t s) {
    const int rows_per_cta = kWarps / d.ks;
    const unsigned grid = (unsigned)((d.ntot + rows_per_cta - 1) / rows_per_cta);
    const size_t smem = (size_t)MT * d.K + kWarps * 2 * MT * sizeof(int);
    return launch_kernel(gemv_dp4a_kernel<MT, T, EPI>, dim3(grid), dim3(kThreads), smem, s, d);
}
// one token, quantizing prologue
template <class T, int EPI, int SRC> cudaError_t launch_dp4a_src_inst(const GemvDev &d, cudaStream_t s) {
    const int rows_per_cta = kWarps / d.ks;
    const unsigned grid = (unsigned)((d.ntot + rows_per_cta - 1) / rows_per_cta);
    size_t smem = (size_t)d.K + kWarps * 2 * sizeof(int);
    if (SRC == SRC_RMSNORM) smem += ((size_t)d.K + 256 + 32) * sizeof(float);
    return launch_kernel(gemv_dp4a_kernel<1, T, EPI, SRC>, dim3(grid), dim3(kThreads), smem, s, d);
}
template <class T, int SRC> cudaError_t launch_dp4a_src(int epi, const GemvDev &d, cudaStream_t s) {
    switch (epi) {
        case EPI_PLAIN: return launch_dp4a_src_inst<T, EPI_PLAIN, SRC>(d, s);
        case EPI_RESIDUAL: return launch_dp4a_src_inst<T, EPI_RESIDUAL, SRC>(d, s);
        case EPI_SWIGLU: return launch_dp4a_src_inst<T, EPI_SWIGLU, SRC>(d, s);
        default: return cudaErrorInvalidValue;
    }
}
template <int MT, class T> cudaError_t launch_dp4a_epi(int epi, const GemvDev &d, cudaStream_t s) {
    switch (epi) {
        case EPI_PLAIN: return launch_dp4a_inst<MT, T, EPI_PLAIN>(d, s);
        case EPI_RESIDUAL: return launch_dp4a_inst<MT, T, EPI_RESIDUAL>(d, s);
        case EPI_SWIGLU: return launch_dp4a_inst<MT, T, EPI_SWIGLU>(d, s);
        case EPI_ACC: return launch_dp4a_inst<MT, T, EPI_ACC>(d, s);
        case EPI_PUSH: return launch_dp4a_inst<MT, T, EPI_PUSH>(d, s);
        default: return cudaErrorInvalidValue;
    }
}
template <class T> cudaError_t launch_dp4a_m(int M, int epi, const GemvDev &d, cudaStream_t s) {
    switch (M) {
        case 1: return launch_dp4a_epi<1, T>(epi, d, s);
        case 2: return launch_dp4a_epi<2, T>(epi, d, s);
        case 3: return launch_dp4a_epi<3, T>(epi, d, s);
        case 4: return launch_dp4a_epi<4, T>(epi, d, s);
        default: return cudaErrorInvalidValue;
    }
}

template <int NT, class T, int EPI> cudaError_t launch_mma_inst(const GemvDev &d, cudaStream_t s) {
    unsigned grid = 0;
    for (int g = 0; g < d.count; ++g) grid += (unsigned)((d.n[g] + 15) / 16);
    return launch_kernel(gemv_mma_kernel<NT, T, EPI>, dim3(grid), dim3(kThreads), (size_t)0, s, d);
}
template <int NT, class T> cudaError_t launch_mma_epi(int epi, const GemvDev &d, cudaStream_t s) {
    switch (epi) {
        case EPI_PLAIN: return launch_mma_inst<NT, T, EPI_PLAIN>(d, s);
        case EPI_RESIDUAL: return launch_mma_inst<NT, T, EPI_RESIDUAL>(d, s);
        case EPI_ACC: return launch_mma_inst<NT, T, EPI_ACC>(d, s);
        case EPI_ARGMAX: return launch_mma_inst<NT, T, EPI_ARGMAX>(d, s);
        case EPI_PUSH: return launch_mma_inst<NT, T, EPI_PUSH>(d, s);
        default: return cudaErrorInvalidValue;
    }
}
template <class T> cudaError_t launch_mma_m(int M, int epi, const GemvDev &d, cudaStream_t s) {
    if (M <= 8) return launch_mma_epi<1, T>(epi, d, s);
    if (M <= 16) return launch_mma_epi<2, T>(epi, d, s);
    if (M <= 32) return launch_mma_epi<4, T>(epi, d, s);
    if (M <= 64) return launch_mma_epi<8, T>(epi, d, s);
    return cudaErrorInvalidValue;
}

template <int MT, class T> cudaError_t set_attr_dp4a() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemv_dp4a_kernel<MT, T, EPI_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDp4aSmem))) return e;
    if ((e = cudaFuncSetAttribute(gemv_dp4a_kernel<MT, T, EPI_RESIDUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDp4aSmem))) return e;
    if ((e = cudaFuncSetAttribute(gemv_dp4a_kernel<MT, T, EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDp4aSmem))) return e;
    if ((e = cudaFuncSetAttribute(gemv_dp4a_kernel<MT, T, EPI_ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDp4aSmem))) return e;
    if ((e = cudaFuncSetAttribute(gemv_dp4a_kernel<MT, T, EPI_PUSH>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDp4aSmem))) return e;
    return cudaSuccess;
}
template <class T, int SRC> cudaError_t set_attr_dp4a_src() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemv_dp4a_kernel<1, T, EPI_PLAIN, SRC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDp4aSmem))) return e;
    if ((e = cudaFuncSetAttribute(gemv_dp4a_kernel<1, T, EPI_RESIDUAL, SRC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDp4aSmem))) return e;
    if ((e = cudaFuncSetAttribute(gemv_dp4a_kernel<1, T, EPI_SWIGLU, SRC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDp4aSmem))) return e;
    return cudaSuccess;
}

}  // namespace

cudaError_t init_gemv() {
    cudaError_t e;
#define W8A8_SET(MT)                                               \
    if ((e = set_attr_dp4a<MT, Bf16>()) != cudaSuccess) return e;  \
    if ((e = set_attr_dp4a<MT, F32>()) != cudaSuccess) return e;
    W8A8_SET(1) W8A8_SET(2) W8A8_SET(3) W8A8_SET(4)
#undef W8A8_SET
    if ((e = set_attr_dp4a_src<Bf16, SRC_WITH_MAX>()) != cudaSuccess) return e;
    if ((e = set_attr_dp4a_src<F32, SRC_WITH_MAX>()) != cudaSuccess) return e;
    if ((e = set_attr_dp4a_src<Bf16, SRC_RMSNORM>()) != cudaSuccess) return e;
    if ((e = set_attr_dp4a_src<F32, SRC_RMSNORM>()) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t launch_gemv_dp4a(const LinearArgs &l, cudaStream_t s) {
    if (l.M < 1 || l.M > 4 || l.K > 24576) return cudaErrorInvalidValue;
    GemvDev d = make_dev(l);
    // Split K over the warps of a CTA while there are too few output channels to fill the GPU.
    const int want = sm_count() * 16;
    int ks = 1;
    while (ks < kWarps && d.ntot * ks < want && l.K / (ks * 2) >= 512) ks *= 2;
    d.ks = ks;
    if (l.src != SRC_CODES) {
        // shared memory: codes + (RMSNorm) the row as float32; 5 bytes per element must fit beside the reductions
        if (l.M != 1 || (l.src == SRC_RMSNORM && l.K > 16384)) return cudaErrorInvalidValue;
        if (l.src == SRC_WITH_MAX)
            return l.dtype == 0 ? launch_dp4a_src<Bf16, SRC_WITH_MAX>(l.epilogue, d, s) : launch_dp4a_src<F32, SRC_WITH_MAX>(l.epilogue, d, s);
        if (l.src == SRC_RMSNORM)
            return l.dtype == 0 ? launch_dp4a_src<Bf16, SRC_RMSNORM>(l.epilogue, d, s) : launch_dp4a_src<F32, SRC_RMSNORM>(l.epilogue, d, s);
        return cudaErrorInvalidValue;
    }
    return l.dtype == 0 ? launch_dp4a_m<Bf16>(l.M, l.epilogue, d, s) : launch_dp4a_m<F32>(l.M, l.epilogue, d, s);
}

cudaError_t launch_argmax_finish(const unsigned long long *partial, int blocks, int M, uint32_t *token, float *value, cudaStream_t s) {
    return launch_kernel(argmax_finish_kernel, dim3(M), dim3(1024), (size_t)0, s, partial, blocks, token, value);
}

cudaError_t launch_gemv_mma(const LinearArgs &l, cudaStream_t s) {
    if (l.M < 1 || l.M > 64 || l.epilogue == EPI_SWIGLU) return cudaErrorInvalidValue;
    GemvDev d = make_dev(l);
    return l.dtype == 0 ? launch_mma_m<Bf16>(l.M, l.epilogue, d, s) : launch_mma_m<F32>(l.M, l.epilogue, d, s);
}

}  // namespace w8a8
