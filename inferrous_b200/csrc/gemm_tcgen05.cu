// Prefill-regime W8A8 projection on the 5th-generation tensor cores (sm_100a only):
// TMA-staged 128-byte-swizzled tiles of the int8 activations [M,K] and weights [N,K],
// tcgen05.mma kind::i8 (s8 x s8 -> s32) accumulating in tensor memory, and a dequantizing
// epilogue read back with tcgen05.ld.
//
// Replaces, from crates/inferrous-qwen3/: linear_large + tma_copy + tma_word
// (src/kernels.rs:1145-1289,154-171,316-320), linear_tiled (:1038-1141), the tensor-map builder
// tensor::map (src/tensor.rs:5-39) and the separate `residual` pass of prefill
// (src/gpu.rs:419-420).  The reference feeds warp-level mma.sync from a single-buffered TMA
// stage; here one persistent CTA per SM runs three specialised roles:
//   warp 0      TMA producer: a ring of {A 128x128 B, B BNx128 B} stages (BN = 256, 128 or 64 output channels per
//               tile; 4, 6 or 8 stages, 192 KiB in flight either way)
//   warp 1      MMA issuer: one elected lane issues 4 x tcgen05.mma (M128 N=BN K32) per stage
//               into one of two BN-column accumulators, and owns the TMEM allocation
//   warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns, (f32(acc)*a_scale[m])*w_scale[n],
//               bf16, optional residual add, 16-byte stores -- overlapped with the next tile
// Every wait on an mbarrier is bounded (about two seconds); on expiry the CTA records a code
// in the device status word, stops issuing work, and leaves through the common exit that
// waits for its own TMA copies and frees its tensor memory.
#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"
#include "gemm_common.cuh"

#include <cstdio>

namespace w8a8 {
namespace {

constexpr int BLOCK_M = 128;   // tokens per tile  (UMMA M)
constexpr int BLOCK_K = 128;   // bytes of K per stage = one 128-byte swizzle atom
constexpr int UMMA_K = 32;     // bytes of K per tcgen05.mma kind::i8
constexpr int A_BYTES = BLOCK_M * BLOCK_K;
constexpr int kThreads = 192;

// Output channels per tile (UMMA N) are a template parameter: 256 when the matrix has enough of them to give every
// SM a tile, 128 or 64 when it does not (O, down and Q|K|V at up to a few hundred tokens).  With few CTAs the kernel
// is bound by the latency of its own TMA round trips, not by the tensor pipe, so narrower tiles on more SMs win
// although each re-reads the activation tile.  Every shape keeps 192 KiB of stages in flight per CTA.
template <int BN> struct Tile {
    static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int kBBytes = BN * BLOCK_K;
    static constexpr int kStageBytes = A_BYTES + kBBytes;
    static constexpr int kTmemCols = 2 * BN;  // two accumulators of BN columns (a power of two >= 32)
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};


template <class T, int EPI, int BLOCK_N>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmDev p) {
    typedef typename T::storage S;
    constexpr int STAGES = Tile<BLOCK_N>::kStages;
    constexpr int B_BYTES = Tile<BLOCK_N>::kBBytes;
    constexpr int STAGE_BYTES = Tile<BLOCK_N>::kStageBytes;
    constexpr int TMEM_COLS = Tile<BLOCK_N>::kTmemCols;
    (void)B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the swizzle pattern of TMA and of the UMMA descriptor is a function
    // of the address bits, and both assume an atom-aligned tile base.
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    uint8_t *gen_tiles = smem_raw + (tiles - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen_tiles + STAGES * STAGE_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) acc_full, [2S+2..2S+4) acc_empty
    const uint32_t bar_base = tiles + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto accf_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto acce_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (p.M + BLOCK_M - 1) / BLOCK_M;
    const int n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
    const int num_tiles = m_tiles * n_tiles;
    const int num_kb = p.K / BLOCK_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(accf_bar(a), 1);
            mbar_init(acce_bar(a), 4);  // one arrival per epilogue warp
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

    dependency_wait();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, WAIT_STAGE_EMPTY))) break;
                    mbar_expect_tx(full_bar(stage), STAGE_BYTES);
                    const uint32_t a_dst = tiles + stage * STAGE_BYTES;
                    tma_load_2d(a_dst, &map_a, kb * BLOCK_K, m_blk * BLOCK_M, full_bar(stage));
                    tma_load_2d(a_dst + A_BYTES, &map_b, kb * BLOCK_K, n_blk * BLOCK_N, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // Abandoned: let the copies already in flight land before the CTA may exit.
                // A stage that was armed completes its phase when its bytes arrive.
                for (int s = 0; s < STAGES; ++s) {
                    const unsigned long long t0 = global_ns();
                    uint32_t par = (s < stage) ? phase : (phase ^ 1u);
                    while (!mbar_try_wait(full_bar(s), par) && global_ns() - t0 < kWaitLimitNs / 4) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BLOCK_M, BLOCK_N);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!(ok = mbar_wait(acce_bar(acc), acc_phase ^ 1u, abort_flag, p.status, WAIT_ACC_EMPTY))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BLOCK_N);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, p.status, WAIT_TMA_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = tiles + stage * STAGE_BYTES;
                    const uint64_t a_desc = smem_desc_sw128(a_addr);
                    const uint64_t b_desc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        // advancing K inside the swizzle atom = advancing the start address
                        const uint64_t koff = (uint64_t)((k * UMMA_K) >> 4);
                        umma_i8(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(accf_bar(acc));  // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, +32) belong to this warp
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
            const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            ok = mbar_wait(accf_bar(acc), acc_phase, abort_flag, p.status, WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int m = m_blk * BLOCK_M + quarter * 32 + lane;
            const bool m_ok = m < p.M;
            const float as = (EPI != EPI_ACC && m_ok) ? p.a_scale[m] : 0.0f;
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BLOCK_N);
            drain_accumulator<T, EPI>(p, t_row, m, m_ok, as, n_blk * BLOCK_N, BLOCK_N);
            // accumulator drained: hand it back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(acc));
        }
    }

    // common exit: every role comes here, whether it finished or gave up
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

cudaError_t load_encode() {
    if (g_encode) return cudaSuccess;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess) return e;
    if (q != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return cudaSuccess;
}

// [rows, K] int8 row-major, box = 128 bytes of K x box_rows rows, 128-byte swizzle, zero fill
// outside the matrix (partial last tiles read zeros, which add nothing to the products).
cudaError_t encode_map_impl(CUtensorMap *map, const void *base, int rows, int K, int box_rows) {
    cudaError_t e = load_encode();
    if (e != cudaSuccess) return e;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <class T, int EPI, int BN> cudaError_t launch_inst(const CUtensorMap &ma, const CUtensorMap &mb, const GemmDev &d, cudaStream_t s) {
    const int tiles = ((d.M + BLOCK_M - 1) / BLOCK_M) * ((d.N + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    return launch_kernel(gemm_tcgen05_kernel<T, EPI, BN>, dim3(grid), dim3(kThreads), (size_t)Tile<BN>::kSmemBytes, s, ma, mb, d);
}
template <class T, int BN> cudaError_t launch_epi(int epi, const CUtensorMap &ma, const CUtensorMap &mb, const GemmDev &d, cudaStream_t s) {
    switch (epi) {
        case EPI_PLAIN: return launch_inst<T, EPI_PLAIN, BN>(ma, mb, d, s);
        case EPI_RESIDUAL: return launch_inst<T, EPI_RESIDUAL, BN>(ma, mb, d, s);
        case EPI_ACC: return launch_inst<T, EPI_ACC, BN>(ma, mb, d, s);
        default: return cudaErrorInvalidValue;
    }
}
template <class T, int EPI, int BN> cudaError_t set_attr() {
    return cudaFuncSetAttribute(gemm_tcgen05_kernel<T, EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Tile<BN>::kSmemBytes);
}
template <class T, int BN> cudaError_t set_attrs() {
    cudaError_t e;
    if ((e = set_attr<T, EPI_PLAIN, BN>()) != cudaSuccess) return e;
    if ((e = set_attr<T, EPI_RESIDUAL, BN>()) != cudaSuccess) return e;
    return set_attr<T, EPI_ACC, BN>();
}

}  // namespace

cudaError_t encode_tile_map(CUtensorMap *map, const void *base, int rows, int K, int box_rows) {
    return encode_map_impl(map, base, rows, K, box_rows);
}

cudaError_t init_gemm_tcgen05() {
    cudaError_t e;
    if ((e = load_encode()) != cudaSuccess) return e;
    if ((e = set_attrs<Bf16, 256>()) != cudaSuccess) return e;
    if ((e = set_attrs<Bf16, 128>()) != cudaSuccess) return e;
    if ((e = set_attrs<Bf16, 64>()) != cudaSuccess) return e;
    if ((e = set_attrs<F32, 256>()) != cudaSuccess) return e;
    if ((e = set_attrs<F32, 128>()) != cudaSuccess) return e;
    if ((e = set_attrs<F32, 64>()) != cudaSuccess) return e;
    return cudaSuccess;
}

// Output channels per tile.  With a tile for (nearly) every SM at 256 channels the kernel is bound by the tensor pipe
// and the widest tile is right.  Below that it is bound by the serial TMA round trips of one tile's K loop, whose
// number is K blocks / stages, i.e. proportional to 1/8, 1/6 and 1/4 for 64, 128 and 256 channels: take the shape
// with the smallest (waves of tiles) x (round trips per tile), the wider one on a tie.
int tcgen05_tile_channels(int M, int N) {
    const int m_tiles = (M + BLOCK_M - 1) / BLOCK_M;
    const int sms = sm_count();
    if (m_tiles * ((N + 255) / 256) >= sms * 3 / 4) return 256;
    int best = 256;
    long long best_cost = -1;
    for (int bn = 256; bn >= 64; bn /= 2) {
        const long long tiles = (long long)m_tiles * ((N + bn - 1) / bn);
        const long long waves = (tiles + sms - 1) / sms;
        const long long cost = waves * (bn == 256 ? 6 : (bn == 128 ? 4 : 3));  // 24 / stages
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

cudaError_t make_weight_maps(w8a8_weight *wt) {
    cudaError_t e = encode_map_impl(&wt->map_rows256, wt->w, wt->N, wt->K, 256);
    if (e != cudaSuccess) return e;
    e = encode_map_impl(&wt->map_rows128, wt->w, wt->N, wt->K, 128);
    if (e != cudaSuccess) return e;
    e = encode_map_impl(&wt->map_rows96, wt->w, wt->N, wt->K, 96);
    if (e != cudaSuccess) return e;
    e = encode_map_impl(&wt->map_rows64, wt->w, wt->N, wt->K, 64);
    if (e != cudaSuccess) return e;
    wt->has_maps = true;
    return cudaSuccess;
}

cudaError_t launch_gemm_tcgen05(const LinearArgs &l, const w8a8_weight *wt, cudaStream_t s) {
    if (!wt || !wt->has_maps || l.count != 1) return cudaErrorInvalidValue;
    // The activation map is encoded on the host per call (a pure function of pointer and shape:
    // no device access, no allocation) and travels as a kernel parameter, so a captured graph
    // keeps its own copy.
    CUtensorMap map_a;
    cudaError_t e = encode_map_impl(&map_a, l.q, l.M, l.K, BLOCK_M);
    if (e != cudaSuccess) return e;
    GemmDev d{};
    d.a_scale = l.a_scale; d.w_scale = wt->w_scale; d.M = l.M; d.N = wt->N; d.K = l.K;
    d.y = l.out[0]; d.residual = l.residual; d.combined = l.combined; d.acc = l.acc;
    d.status = device_status_ptr();
    switch (tcgen05_tile_channels(l.M, wt->N)) {
        case 256:
            return l.dtype == 0 ? launch_epi<Bf16, 256>(l.epilogue, map_a, wt->map_rows256, d, s)
                                : launch_epi<F32, 256>(l.epilogue, map_a, wt->map_rows256, d, s);
        case 128:
            return l.dtype == 0 ? launch_epi<Bf16, 128>(l.epilogue, map_a, wt->map_rows128, d, s)
                                : launch_epi<F32, 128>(l.epilogue, map_a, wt->map_rows128, d, s);
        default:
            return l.dtype == 0 ? launch_epi<Bf16, 64>(l.epilogue, map_a, wt->map_rows64, d, s)
                                : launch_epi<F32, 64>(l.epilogue, map_a, wt->map_rows64, d, s);
    }
}

}  // namespace w8a8
