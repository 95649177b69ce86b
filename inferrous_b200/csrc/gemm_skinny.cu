// Few-token W8A8 projection on the tcgen05 tensor cores (sm_100a): 5..256 tokens, where the
// product is bound by the one pass over the int8 weights, not by the MMA rate.
//
// Replaces, from crates/inferrous-qwen3/src/kernels.rs: linear_splitk (:935-1034, 2..31 rows),
// linear_tiled (:1038-1141, 32..255 rows) and their host dispatch (src/gpu.rs:473-494).
// The reference tiles tokens x channels for warp-level mma.sync.  Here the roles of the operands
// are swapped so that a tile never wastes MMA rows on absent tokens: the WEIGHTS are the MMA's
// M side (128 output channels per tile), the tokens its N side (padded to a multiple of 16), and
// the whole K extent of a tile streams through a deep TMA ring:
//   warp 0      TMA producer: per 128-byte K block one 128x128 B weight box and one NTOKx128 B
//               activation box (both 128-byte swizzled, K-major)
//   warp 1      MMA issuer: 4 x tcgen05.mma kind::i8 (M128, N=NTOK, K32) per stage into one of two
//               tensor-memory accumulators; owns the TMEM allocation
//   warps 2-5   epilogue: tcgen05.ld (lane = channel, column = token), dequantize, bf16, stores
// Work is split stream-K style: the (tile, K block) pairs are laid out in one line and cut into
// equal contiguous spans, one per SM, so every SM streams the same number of weight bytes
// whatever N is.  A span that ends inside a tile adds its int32 partial sums into a per-device
// scratch tile with red.global.add (exact, order-free) and bumps an arrival counter; whoever
// completes the count reads the sums back, runs the epilogue and returns scratch and counter
// to zero.  Nobody waits on anybody: there is no spin on another CTA's progress.
// Every mbarrier wait is bounded (ptx.cuh).
#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"

#include <mutex>

namespace w8a8 {
namespace {

constexpr int TILE_N = 128;    // output channels per tile (UMMA M)
constexpr int BLOCK_K = 128;   // bytes of K per stage
constexpr int UMMA_K = 32;
constexpr int A_BYTES = TILE_N * BLOCK_K;
constexpr int kThreads = 192;
constexpr int kSmemBudget = 216 * 1024;
constexpr int TMEM_COLS = 512;

struct SkinnyDev {
    const float *a_scale;
    const float *w_scale;
    int M, N, K, ntok;   // ntok = tokens padded to a multiple of 16
    int stages;
    int kps;             // 128-byte K blocks per stage (1, 2 or 4): wider stages keep DRAM pages open
    void *y;
    const void *residual;
    void *combined;
    int32_t *acc;
    int32_t *scratch;     // [grid][4 quarters][kSkinnyMaxTokens][32]
    uint32_t *counters;   // [grid][4]
    uint32_t *status;
};

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// First unit of CTA c when `units` are cut into `grid` contiguous spans.
__device__ __forceinline__ long long span_begin(long long c, long long units, int grid) { return c * units / grid; }

template <class T, int EPI>
__device__ __forceinline__ void finish_value(const SkinnyDev &p, int m, int n, int acc, float ws) {
    typedef typename T::storage S;
    const int64_t o = (int64_t)m * p.N + n;
    if (EPI == EPI_ACC) {
        p.acc[o] = acc;
        return;
    }
    const float y = dequant(acc, p.a_scale[m], ws);
    if (p.y) T::store(static_cast<S *>(p.y) + o, y);
    if (EPI == EPI_RESIDUAL) {
        const float r = T::load(static_cast<const S *>(p.residual) + o);
        T::store(static_cast<S *>(p.combined) + o, bf16_rne(__fadd_rn(r, y)));
    }
}

template <class T, int EPI, int TOK_STRIDE = kSkinnyMaxTokens>
__global__ void __launch_bounds__(kThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q, const SkinnyDev p) {
    extern __shared__ uint8_t smem_raw[];
    const int NS = p.stages;
    const int KPS = p.kps;
    const int b_bytes = p.ntok * BLOCK_K;
    const int stage_bytes = KPS * (A_BYTES + b_bytes);  // multiple of 1024: ntok is a multiple of 16
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (tiles - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + (size_t)NS * stage_bytes);
    const uint32_t bar_base = tiles + (uint32_t)(NS * stage_bytes);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (NS + s); };
    auto accf_bar = [&](int a) { return bar_base + 8u * (2 * NS + a); };
    auto acce_bar = [&](int a) { return bar_base + 8u * (2 * NS + 2 + a); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * NS + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (p.N + TILE_N - 1) / TILE_N;
    const int num_kb = p.K / (BLOCK_K * KPS);  // K groups (stages) per tile
    const long long units = (long long)n_tiles * num_kb;
    const long long u_begin = span_begin(blockIdx.x, units, gridDim.x);
    const long long u_end = span_begin(blockIdx.x + 1, units, gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(accf_bar(a), 1);
            mbar_init(acce_bar(a), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true, waited = false;
        for (long long u = u_begin; u < u_end && ok; ++u) {
            const int tile = (int)(u / num_kb), kb = (int)(u % num_kb);
            if (lane == 0) ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, WAIT_STAGE_EMPTY);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane == 0) {
                mbar_expect_tx(full_bar(stage), (uint32_t)stage_bytes);
                const uint32_t dst = tiles + (uint32_t)(stage * stage_bytes);
                // weights are immutable: their copies may start before the predecessor kernel is done
                for (int j = 0; j < KPS; ++j)
                    tma_load_2d(dst + (uint32_t)(j * A_BYTES), &map_w, (kb * KPS + j) * BLOCK_K, tile * TILE_N, full_bar(stage));
                if (!waited) {
                    dependency_wait();
                    waited = true;
                }
                for (int j = 0; j < KPS; ++j)
                    tma_load_2d(dst + (uint32_t)(KPS * A_BYTES + j * b_bytes), &map_q, (kb * KPS + j) * BLOCK_K, 0, full_bar(stage));
            }
            if (++stage == NS) { stage = 0; phase ^= 1u; }
        }
        if (!ok && lane == 0) {
            for (int s = 0; s < NS; ++s) {
                const unsigned long long t0 = global_ns();
                const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
                while (!mbar_try_wait(full_bar(s), par) && global_ns() - t0 < kWaitLimitNs / 4) {}
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(TILE_N, p.ntok);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (long long u = u_begin; u < u_end && ok; ++it) {
                const int kb0 = (int)(u % num_kb);
                const int kbn = (int)min((long long)(num_kb - kb0), u_end - u);  // K blocks of this segment
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!(ok = mbar_wait(acce_bar(acc), acc_phase ^ 1u, abort_flag, p.status, WAIT_ACC_EMPTY))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 256);
                for (int i = 0; i < kbn; ++i) {
                    if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, p.status, WAIT_TMA_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = tiles + (uint32_t)(stage * stage_bytes);
                    for (int j = 0; j < KPS; ++j) {
                        const uint64_t a_desc = smem_desc_sw128(a_addr + (uint32_t)(j * A_BYTES));
                        const uint64_t b_desc = smem_desc_sw128(a_addr + (uint32_t)(KPS * A_BYTES + j * b_bytes));
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                            const uint64_t koff = (uint64_t)((k * UMMA_K) >> 4);
                            umma_i8(d_tmem, a_desc + koff, b_desc + koff, idesc, (i | j | k) != 0 ? 1u : 0u);
                        }
                    }
                    umma_commit(empty_bar(stage));
                    if (++stage == NS) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(accf_bar(acc));
                u += kbn;
            }
        }
    } else {
        // ---------------- epilogue warps: lane = output channel, column = token ----------------
        dependency_wait();
        const int quarter = warp & 3;
        int it = 0;
        bool ok = true;
        for (long long u = u_begin; u < u_end && ok; ++it) {
            const int tile = (int)(u / num_kb), kb0 = (int)(u % num_kb);
            const int kbn = (int)min((long long)(num_kb - kb0), u_end - u);
            u += kbn;
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            ok = mbar_wait(accf_bar(acc), acc_phase, abort_flag, p.status, WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int n = tile * TILE_N + quarter * 32 + lane;
            const bool n_ok = n < p.N;
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 256);
            const bool whole = (kbn == num_kb);
            const float ws = (EPI != EPI_ACC && n_ok) ? p.w_scale[n] : 0.0f;

            // which scratch tile a split tile uses: the id of the CTA whose span holds the tile's first K block
            int slot = 0;
            if (!whole) {
                const long long first = (long long)tile * num_kb;
                long long c = ((first + 1) * gridDim.x - 1) / units;
                while (c > 0 && span_begin(c, units, gridDim.x) > first) --c;
                while (span_begin(c + 1, units, gridDim.x) <= first) ++c;
                slot = (int)c;
            }
            int32_t *sc = p.scratch + ((size_t)slot * 4 + quarter) * ((size_t)TOK_STRIDE * 32);

            for (int c0 = 0; c0 < p.ntok; c0 += 16) {
                int v[16];
                tmem_ld_32x16(t_row + (uint32_t)c0, v);
                tmem_ld_wait();
                if (whole) {
                    if (n_ok) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (c0 + i < p.M) finish_value<T, EPI>(p, c0 + i, n, v[i], ws);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (c0 + i < p.M) atomicAdd(sc + (c0 + i) * 32 + lane, v[i]);  // result unused: a reduction
                }
            }
            // accumulator drained: hand it back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(acc));

            if (!whole) {
                // publish, count arrivals, and let the last contributor of this quarter finish it
                __threadfence();
                __syncwarp();
                uint32_t prev = 0;
                uint32_t *cnt = p.counters + (size_t)slot * 4 + quarter;
                if (lane == 0) prev = atomicAdd(cnt, (uint32_t)kbn);
                prev = __shfl_sync(0xffffffffu, prev, 0);
                if (prev + (uint32_t)kbn == (uint32_t)num_kb) {
                    __threadfence();
                    for (int m0 = 0; m0 < p.M; m0 += 8) {  // eight independent L2 reads in flight
                        int sums[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) sums[i] = (m0 + i < p.M) ? __ldcg(sc + (m0 + i) * 32 + lane) : 0;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (m0 + i < p.M) {
                                sc[(m0 + i) * 32 + lane] = 0;
                                if (n_ok) finish_value<T, EPI>(p, m0 + i, n, sums[i], ws);
                            }
                    }
                    if (lane == 0) *cnt = 0;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <class T, int EPI> cudaError_t launch_inst(const CUtensorMap &mw, const CUtensorMap &mq, const SkinnyDev &d, int grid,
                                                    size_t smem, cudaStream_t s) {
    return launch_kernel(gemm_skinny_kernel<T, EPI>, dim3(grid), dim3(kThreads), smem, s, mw, mq, d);
}
template <class T> cudaError_t launch_epi(int epi, const CUtensorMap &mw, const CUtensorMap &mq, const SkinnyDev &d, int grid,
                                          size_t smem, cudaStream_t s) {
    switch (epi) {
        case EPI_PLAIN: return launch_inst<T, EPI_PLAIN>(mw, mq, d, grid, smem, s);
        case EPI_RESIDUAL: return launch_inst<T, EPI_RESIDUAL>(mw, mq, d, grid, smem, s);
        case EPI_ACC: return launch_inst<T, EPI_ACC>(mw, mq, d, grid, smem, s);
        default: return cudaErrorInvalidValue;
    }
}
template <class T, int EPI> cudaError_t set_attr() {
    return cudaFuncSetAttribute(gemm_skinny_kernel<T, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 2048);
}

// K blocks per stage and ring depth: the widest stage (4, 2 or 1 blocks of 128 bytes, wider stages keep DRAM pages
// open) that divides K and still leaves a ring of at least three stages in shared memory.
bool pick_stages(int K, int ntok, int &kps, int &stages) {
    kps = 4;
    while (kps > 1 && ((K / BLOCK_K) % kps != 0 || (kSmemBudget - 1024) / (kps * (A_BYTES + ntok * BLOCK_K)) < 3)) kps /= 2;
    stages = (kSmemBudget - 1024) / (kps * (A_BYTES + ntok * BLOCK_K));
    if (stages > 16) stages = 16;
    return stages >= 2;
}

}  // namespace

cudaError_t init_gemm_skinny() {
    cudaError_t e;
    if ((e = set_attr<Bf16, EPI_PLAIN>()) != cudaSuccess) return e;
    if ((e = set_attr<Bf16, EPI_RESIDUAL>()) != cudaSuccess) return e;
    if ((e = set_attr<Bf16, EPI_ACC>()) != cudaSuccess) return e;
    if ((e = set_attr<F32, EPI_PLAIN>()) != cudaSuccess) return e;
    if ((e = set_attr<F32, EPI_RESIDUAL>()) != cudaSuccess) return e;
    if ((e = set_attr<F32, EPI_ACC>()) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t launch_gemm_skinny(const LinearArgs &l, const w8a8_weight *wt, cudaStream_t s) {
    if (!wt || !wt->has_maps || l.count != 1 || l.M < 1 || l.M > kSkinnyMaxTokens) return cudaErrorInvalidValue;
    if (!skinny_scratch() || !skinny_counters()) return cudaErrorInitializationError;
    const int ntok = (l.M + 15) / 16 * 16;
    CUtensorMap map_q;
    cudaError_t e = encode_tile_map(&map_q, l.q, l.M, l.K, ntok);
    if (e != cudaSuccess) return e;
    SkinnyDev d{};
    d.a_scale = l.a_scale; d.w_scale = wt->w_scale; d.M = l.M; d.N = wt->N; d.K = l.K; d.ntok = ntok;
    if (!pick_stages(l.K, ntok, d.kps, d.stages)) return cudaErrorInvalidValue;
    const int kps = d.kps, stages = d.stages;
    const int stage_bytes = kps * (A_BYTES + ntok * BLOCK_K);
    d.y = l.out[0]; d.residual = l.residual; d.combined = l.combined; d.acc = l.acc;
    d.scratch = skinny_scratch(); d.counters = skinny_counters(); d.status = device_status_ptr();
    const long long units = (long long)((wt->N + TILE_N - 1) / TILE_N) * (l.K / (BLOCK_K * kps));
    const int grid = (int)(units < sm_count() ? units : sm_count());
    const size_t smem = (size_t)stages * stage_bytes + 1024 + 8 * (2 * (size_t)stages + 4) + 64;
    return l.dtype == 0 ? launch_epi<Bf16>(l.epilogue, wt->map_rows128, map_q, d, grid, smem, s)
                        : launch_epi<F32>(l.epilogue, wt->map_rows128, map_q, d, grid, smem, s);
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant: the stream-K scratch lives in a fixed device array of this module.
// ---------------------------------------------------------------------------------------
namespace {

constexpr int kStaticMaxTokens = 16;   // token limit of the allocation-free entry point
constexpr int kStaticSlots = 160;      // CTAs (one scratch tile each); the grid is capped to this
constexpr size_t kStaticTileInts = (size_t)kStaticSlots * 4 * kStaticMaxTokens * 32;
constexpr size_t kStaticCounterInts = (size_t)kStaticSlots * 4;
constexpr size_t kStaticClearInts = kStaticTileInts + kStaticCounterInts;  // what every call returns to zero
constexpr size_t kStaticInts = kStaticClearInts + 2 /* status words */ + 62 /* pad */;

// 1.25 MiB, resident on every GPU that loads the library until the process exits.
// In host code this name is only a stand-in for the symbol: the device address comes from
// cudaGetSymbolAddress (static_scratch_address below) and that pointer is what kernels receive.
static __device__ __align__(256) int32_t g_static_scratch[kStaticInts];

struct StaticState {
    bool ready = false;
    int32_t *base = nullptr;
    int sms = 0;
};
StaticState g_static[64];
std::mutex g_static_mu;  // two host threads may make their first call on a device at the same time

// Once per device, with that device current: resolve the array's device address and raise the
// kernels' shared-memory limit.  Neither call allocates.
cudaError_t static_setup(int dev) {
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticState &st = g_static[dev];
    if (st.ready) return cudaSuccess;
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&st.sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(gemm_skinny_kernel<Bf16, EPI_PLAIN, kStaticMaxTokens>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kSmemBudget + 2048)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(gemm_skinny_kernel<F32, EPI_PLAIN, kStaticMaxTokens>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kSmemBudget + 2048)) != cudaSuccess) return e;
    st.base = static_cast<int32_t *>(ptr);
    st.ready = true;
    return cudaSuccess;
}

}  // namespace

// See w8a8_linear_no_alloc in include/w8a8.h.  Returns cudaErrorInvalidValue for shapes beyond the
// fixed scratch (the C ABI turns that into W8A8_ERR_UNSUPPORTED before coming here).
cudaError_t launch_linear_no_alloc(const int8_t *q, const float *a_scale, const int8_t *w, const float *w_scale, int M, int N,
                                   int K, void *y, int dtype, cudaStream_t s) {
    if (M < 1 || M > kStaticMaxTokens || N < 1 || K < BLOCK_K || K % BLOCK_K != 0) return cudaErrorInvalidValue;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if ((e = static_setup(dev)) != cudaSuccess) return e;
    const StaticState &st = g_static[dev];

    // Tensor maps are encoded on the host (no device work, no allocation) and passed by value.
    CUtensorMap map_w, map_q;
    const int ntok = kStaticMaxTokens;
    if ((e = encode_tile_map(&map_w, w, N, K, TILE_N)) != cudaSuccess) return e;
    if ((e = encode_tile_map(&map_q, q, M, K, ntok)) != cudaSuccess) return e;

    SkinnyDev d{};
    d.a_scale = a_scale; d.w_scale = w_scale; d.M = M; d.N = N; d.K = K; d.ntok = ntok;
    if (!pick_stages(K, ntok, d.kps, d.stages)) return cudaErrorInvalidValue;  // the same rule as the regular launcher
    const int kps = d.kps, stages = d.stages;
    const int stage_bytes = kps * (A_BYTES + ntok * BLOCK_K);
    d.y = y;
    d.scratch = st.base;
    d.counters = reinterpret_cast<uint32_t *>(st.base + kStaticTileInts);
    d.status = reinterpret_cast<uint32_t *>(st.base + kStaticTileInts + kStaticCounterInts);
    // The array keeps whatever the previous call left (normally zeros, but not after an abandoned
    // launch): partial tiles and counters must start at zero, so clear them in stream order.  The
    // status words behind them are NOT cleared here: a wait that ran out stays on record until
    // w8a8_device_status reads it.
    if ((e = cudaMemsetAsync(st.base, 0, kStaticClearInts * sizeof(int32_t), s)) != cudaSuccess) return e;

    const long long units = (long long)((N + TILE_N - 1) / TILE_N) * (K / (BLOCK_K * kps));
    int grid = st.sms < kStaticSlots ? st.sms : kStaticSlots;
    if (units < grid) grid = (int)units;
    const size_t smem = (size_t)stages * stage_bytes + 1024 + 8 * (2 * (size_t)stages + 4) + 64;
    if (dtype == 0)
        gemm_skinny_kernel<Bf16, EPI_PLAIN, kStaticMaxTokens><<<grid, kThreads, smem, s>>>(map_w, map_q, d);
    else
        gemm_skinny_kernel<F32, EPI_PLAIN, kStaticMaxTokens><<<grid, kThreads, smem, s>>>(map_w, map_q, d);
    return cudaGetLastError();
}

// The status words of the allocation-free entry point on the current device, read and cleared in stream order
// (no allocation: the copy lands in the caller's host words).  *present = false when that entry point has never
// run on the device.
cudaError_t read_no_alloc_status(cudaStream_t s, uint32_t out[2], bool *present) {
    *present = false;
    out[0] = out[1] = 0;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaSuccess;
    int32_t *words = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        if (!g_static[dev].ready) return cudaSuccess;
        words = g_static[dev].base + kStaticClearInts;
    }
    *present = true;
    if ((e = cudaMemcpyAsync(out, words, 8, cudaMemcpyDeviceToHost, s)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(words, 0, 8, s)) != cudaSuccess) return e;
    return cudaStreamSynchronize(s);
}

}  // namespace w8a8
