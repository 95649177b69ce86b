// Decode-regime W8A8 projection for 2..16 tokens (HBM-bound): whole weight rows stream through a
// shared-memory ring as large bulk copies, warp-level int8 MMAs read their fragments from there.
//
// Replaces, from crates/inferrous-qwen3/src/kernels.rs: linear_splitk (:935-1034) and, for a few
// tokens, linear_pair / linear_triple (:698-806) and linear_residual (:579-618).
// Why this shape: on B200 a weight stream runs fastest when DRAM sees long contiguous runs (a whole
// 4 KiB row at a time) and when many bytes are in flight per SM without holding registers for them;
// bulk asynchronous copies give both, provided each request is large (>= 4 KiB: smaller requests are
// rate-limited per SM).
//   warp 8      producer: a stage is a block of <= 16 output channels x one piece (<= 4096 bytes) of K;
//               lane r issues the bulk copy of channel r's piece into a shared-memory row whose pitch
//               (piece + 64) makes the consumers' 16-byte fragment reads bank-conflict free.  Weights
//               are immutable, so the producer starts before griddepcontrol.wait.
//   warps 0-7   consumers: warp w owns the w-th eighth of every piece (split-K); lane (g,t) reads rows
//               g and g+8 sixteen bytes at a time straight into the A fragments of
//               mma.sync.m16n8k32.s8 (K is consumed in a permuted order, which integer accumulation
//               allows); tokens are the MMA's N side, their fragments cached in registers when the
//               matrix has a single piece.  After the last piece of a block the warps leave their
//               int32 partials in shared memory, meet at a bounded mbarrier, and all 256 threads
//               finish the block: exact sum, dequantize, bf16, optional residual.
// One CTA per SM owns a contiguous, balanced range of output channels (balanced to the channel).
#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace w8a8 {
namespace {

constexpr int kConsumers = 8;
constexpr int kThreads = (kConsumers + 1) * 32;
constexpr int kBlockRows = 16;      // output channels per block = MMA M
constexpr int kMaxPiece = 4096;     // bytes of K per stage row
constexpr int kSmemBudget = 220 * 1024;

struct RowsDev {
    const int8_t *q;
    const float *a_scale;
    int M, K, count;
    const int8_t *w[kMaxGroup];
    const float *ws[kMaxGroup];
    void *out[kMaxGroup];
    int n[kMaxGroup];
    int ntot;
    int piece;    // bytes of K per stage row (multiple of 128)
    int stages;
    const void *residual;
    void *combined;
    int32_t *acc;
    uint32_t *status;
};

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void locate(const RowsDev &a, int row, int &g, int &c) {
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

// NT tiles of 8 tokens.  CACHE: the token fragments of the (single) piece live in registers.
template <int NT, bool CACHE, class T, int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemv_rows_kernel(const RowsDev a) {
    typedef typename T::storage S;
    constexpr int kPartInts = kConsumers * NT * 4 * 32;
    constexpr int kSteps = kMaxPiece / kConsumers / 128;  // 128-byte MMA steps per warp per piece (4)
    extern __shared__ __align__(128) uint8_t smem[];
    const int K = a.K, NS = a.stages, piece = a.piece;
    const int pitch = piece + 64;
    const int stage_bytes = kBlockRows * pitch;
    int *part = reinterpret_cast<int *>(smem + (size_t)NS * stage_bytes);  // [2][kPartInts]
    uint64_t *bars = reinterpret_cast<uint64_t *>(part + 2 * kPartInts);
    const uint32_t ring = smem_u32(smem);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (NS + s); };
    const uint32_t cta_bar = bar_base + 8u * (2 * NS);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * NS + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row_begin = (int)((int64_t)blockIdx.x * a.ntot / gridDim.x);
    const int row_end = (int)((int64_t)(blockIdx.x + 1) * a.ntot / gridDim.x);
    const int npieces = (K + piece - 1) / piece;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), kConsumers);
        }
        mbar_init(cta_bar, kConsumers);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumers) {
        // ---------------- producer warp: lane r copies channel r of the block ----------------
        uint32_t g = 0;  // running stage number; slot = g % NS, phase = (g / NS) & 1
        bool ok = true;
        for (int b0 = row_begin; b0 < row_end && ok; b0 += kBlockRows) {
            const int nr = min(kBlockRows, row_end - b0);
            const int8_t *src = nullptr;
            if (lane < nr) {
                int gi, c;
                locate(a, b0 + lane, gi, c);
                src = a.w[gi] + (int64_t)c * K;
            }
            for (int p = 0; p < npieces; ++p, ++g) {
                const int slot = (int)(g % (uint32_t)NS);
                const uint32_t phase = (g / (uint32_t)NS) & 1u;
                const int len = min(piece, K - p * piece);
                if (lane == 0) {
                    ok = mbar_wait(empty_bar(slot), phase ^ 1u, abort_flag, a.status, WAIT_STAGE_EMPTY);
                    if (ok) mbar_expect_tx(full_bar(slot), (uint32_t)(nr * len));
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                if (lane < nr)
                    bulk_load(ring + (uint32_t)(slot * stage_bytes + lane * pitch), src + (size_t)p * piece, (uint32_t)len, full_bar(slot));
            }
        }
        if (!ok && lane == 0) {  // abandoned: let the copies already in flight land before the CTA may exit
            for (int s = 0; s < NS; ++s) {
                const unsigned long long t0 = global_ns();
                const uint32_t cur = (g / (uint32_t)NS) & 1u;
                const uint32_t par = ((uint32_t)s < g % (uint32_t)NS) ? cur : (cur ^ 1u);
                while (!mbar_try_wait(full_bar(s), par) && global_ns() - t0 < kWaitLimitNs / 4) {}
            }
        }
    } else {
        // ---------------- consumer warps ----------------
        const int gq = lane >> 2, t = lane & 3;
        const int sub = piece / kConsumers;              // bytes of a piece owned by this warp (multiple of 16)
        const int nsteps = (sub + 127) / 128;            // <= kSteps
        dependency_wait();

        // token fragments for (piece p, step s, half h): 16 bytes of token 8j+gq at K offset p*piece + warp*sub + s*128 + h*64 + t*16
        auto load_b = [&](int p, int s, int h, int j) -> uint4 {
            const int tok = j * 8 + gq;
            const int koff = s * 128 + h * 64 + t * 16;
            if (tok < a.M && koff < sub && p * piece + warp * sub + koff < K)
                return *reinterpret_cast<const uint4 *>(a.q + (int64_t)tok * K + (int64_t)p * piece + warp * sub + koff);
            return make_uint4(0, 0, 0, 0);
        };
        uint4 bcache[CACHE ? kSteps : 1][2][NT];
        if (CACHE) {
#pragma unroll
            for (int s = 0; s < kSteps; ++s)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < NT; ++j) bcache[s][h][j] = load_b(0, s, h, j);
        }

        uint32_t cphase = 0, gbase = 0;
        int buf = 0;
        bool ok = true;
        for (int b0 = row_begin; b0 < row_end && ok; b0 += kBlockRows, gbase += (uint32_t)npieces) {
            const int nr = min(kBlockRows, row_end - b0);
            int acc[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[j][i] = 0;

            for (int p = 0; p < npieces; ++p) {
                const uint32_t g = gbase + (uint32_t)p;
                const int slot = (int)(g % (uint32_t)NS);
                const uint32_t phase = (g / (uint32_t)NS) & 1u;
                ok = mbar_wait(full_bar(slot), phase, abort_flag, a.status, WAIT_TMA_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const int len = min(piece, K - p * piece);
                const uint8_t *lo = smem + (size_t)slot * stage_bytes + (size_t)gq * pitch + warp * sub + t * 16;
                const uint8_t *hi = lo + 8 * pitch;
#pragma unroll
                for (int s = 0; s < kSteps; ++s) {
                    if (s < nsteps) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int koff = s * 128 + h * 64;
                            if (koff < sub && warp * sub + koff < len) {  // warp-uniform
                                const uint4 r = *reinterpret_cast<const uint4 *>(lo + koff);
                                const uint4 v = *reinterpret_cast<const uint4 *>(hi + koff);
#pragma unroll
                                for (int j = 0; j < NT; ++j) {
                                    const uint4 b = CACHE ? bcache[CACHE ? s : 0][h][j] : load_b(p, s, h, j);
                                    mma_s8(acc[j], r.x, v.x, r.y, v.y, b.x, b.y);
                                    mma_s8(acc[j], r.z, v.z, r.w, v.w, b.z, b.w);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(slot));  // this warp is done with the stage
            }
            if (!ok) break;

            int *mine = part + buf * kPartInts + warp * (NT * 4 * 32);
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) mine[(j * 4 + i) * 32 + lane] = acc[j][i];
            __syncwarp();
            if (lane == 0) mbar_arrive(cta_bar);
            ok = mbar_wait(cta_bar, cphase, abort_flag, a.status, WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            cphase ^= 1u;
            if (!ok) break;

            const int *src = part + buf * kPartInts;
            for (int idx = tid; idx < NT * 128; idx += kConsumers * 32) {
                int sum = 0;
#pragma unroll
                for (int w = 0; w < kConsumers; ++w) sum += src[w * (NT * 4 * 32) + idx];
                const int l = idx & 31, reg = (idx >> 5) & 3, j = idx >> 7;
                const int r = (l >> 2) + 8 * (reg >> 1);
                const int tok = j * 8 + 2 * (l & 3) + (reg & 1);
                if (r >= nr || tok >= a.M) continue;
                int gi, c;
                locate(a, b0 + r, gi, c);
                const int64_t o = (int64_t)tok * a.n[gi] + c;
                if (EPI == EPI_ACC) {
                    a.acc[o] = sum;
                    continue;
                }
                const float y = dequant(sum, a.a_scale[tok], a.ws[gi][c]);
                if (a.out[gi]) T::store(static_cast<S *>(a.out[gi]) + o, y);
                if (EPI == EPI_RESIDUAL) {
                    const float res = T::load(static_cast<const S *>(a.residual) + o);
                    T::store(static_cast<S *>(a.combined) + o, bf16_rne(__fadd_rn(res, y)));
                }
            }
            buf ^= 1;
        }
    }
    __syncthreads();  // common exit: every role arrives here, finished or abandoned
}

struct Geometry {
    int piece, stages;
    size_t smem;
};
Geometry geometry(int K, int NT) {
    Geometry g;
    g.piece = K < kMaxPiece ? K : kMaxPiece;
    const size_t stage = (size_t)kBlockRows * (g.piece + 64);
    const size_t fixed = 2 * (size_t)kConsumers * NT * 4 * 32 * sizeof(int) + 128;
    int stages = (int)((kSmemBudget - fixed - 1024) / stage);
    if (stages > 24) stages = 24;
    g.stages = stages;
    g.smem = (size_t)stages * stage + fixed + 8 * (2 * (size_t)stages + 2);
    return g;
}

template <int NT, bool CACHE, class T, int EPI> cudaError_t launch_inst(const RowsDev &d, size_t smem, cudaStream_t s) {
    const int grid = d.ntot < sm_count() ? d.ntot : sm_count();
    return launch_kernel(gemv_rows_kernel<NT, CACHE, T, EPI>, dim3(grid), dim3(kThreads), smem, s, d);
}
template <int NT, bool CACHE, class T> cudaError_t launch_epi(int epi, const RowsDev &d, size_t smem, cudaStream_t s) {
    switch (epi) {
        case EPI_PLAIN: return launch_inst<NT, CACHE, T, EPI_PLAIN>(d, smem, s);
        case EPI_RESIDUAL: return launch_inst<NT, CACHE, T, EPI_RESIDUAL>(d, smem, s);
        case EPI_ACC: return launch_inst<NT, CACHE, T, EPI_ACC>(d, smem, s);
        default: return cudaErrorInvalidValue;
    }
}
template <class T> cudaError_t launch_nt(int M, bool cache, int epi, const RowsDev &d, size_t smem, cudaStream_t s) {
    if (M <= 8) return cache ? launch_epi<1, true, T>(epi, d, smem, s) : launch_epi<1, false, T>(epi, d, smem, s);
    if (M <= 16) return cache ? launch_epi<2, true, T>(epi, d, smem, s) : launch_epi<2, false, T>(epi, d, smem, s);
    return cudaErrorInvalidValue;
}

template <int NT, bool CACHE, class T> cudaError_t prime_epi() {
    cudaError_t e;
    const int lim = kSmemBudget + 2048;
    if ((e = cudaFuncSetAttribute(gemv_rows_kernel<NT, CACHE, T, EPI_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim))) return e;
    if ((e = cudaFuncSetAttribute(gemv_rows_kernel<NT, CACHE, T, EPI_RESIDUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim))) return e;
    if ((e = cudaFuncSetAttribute(gemv_rows_kernel<NT, CACHE, T, EPI_ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim))) return e;
    return cudaSuccess;
}
template <class T> cudaError_t prime_t() {
    cudaError_t e;
    if ((e = prime_epi<1, true, T>())) return e;
    if ((e = prime_epi<1, false, T>())) return e;
    if ((e = prime_epi<2, true, T>())) return e;
    if ((e = prime_epi<2, false, T>())) return e;
    return cudaSuccess;
}

}  // namespace

cudaError_t init_gemv_rows() {
    cudaError_t e;
    if ((e = prime_t<Bf16>())) return e;
    if ((e = prime_t<F32>())) return e;
    return cudaSuccess;
}

cudaError_t launch_gemv_rows(const LinearArgs &l, cudaStream_t s) {
    if (l.M < 1 || l.M > 16 || l.K % 128 != 0 || l.epilogue == EPI_SWIGLU) return cudaErrorInvalidValue;
    RowsDev d{};
    d.q = l.q; d.a_scale = l.a_scale; d.M = l.M; d.K = l.K; d.count = l.count;
    int ntot = 0;
    for (int g = 0; g < kMaxGroup; ++g) {
        d.w[g] = l.w[g]; d.ws[g] = l.ws[g]; d.out[g] = l.out[g]; d.n[g] = l.n[g];
        if (g < l.count) ntot += l.n[g];
    }
    d.ntot = ntot;
    const int nt = l.M <= 8 ? 1 : 2;
    const Geometry geo = geometry(l.K, nt);
    if (geo.stages < 2) return cudaErrorInvalidValue;
    d.piece = geo.piece; d.stages = geo.stages;
    d.residual = l.residual; d.combined = l.combined; d.acc = l.acc;
    d.status = device_status_ptr();
    const bool cache = l.K <= kMaxPiece;  // a single piece: token fragments stay in registers
    return l.dtype == 0 ? launch_nt<Bf16>(l.M, cache, l.epilogue, d, geo.smem, s) : launch_nt<F32>(l.M, cache, l.epilogue, d, geo.smem, s);
}

}  // namespace w8a8
