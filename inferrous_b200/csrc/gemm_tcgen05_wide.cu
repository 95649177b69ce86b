// Prefill-regime W8A8 projection with 256x256 output tiles per CTA (sm_100a): the variant of
// gemm_tcgen05.cu for many tokens, where the 128x256 tile is limited by operand traffic from L2
// (48 KiB of operands per 512 MMA cycles).  A 256x256 tile needs 64 KiB per 1024 MMA cycles, a third
// less per multiply; the price is that the two 256-column accumulators fill tensor memory, so the
// epilogue of a tile is not overlapped with the next tile's MMAs (eight epilogue warps keep it short).
//
// Replaces the same reference kernels as gemm_tcgen05.cu (linear_large, src/kernels.rs:1145-1289).
//   warp 0      TMA producer: 3-stage ring of {A 2 x (128x128 B), B 256x128 B}
//   warp 1      MMA issuer: per stage 4 K-steps x 2 tcgen05.mma (M128 N256 K32), one per token half
//   warps 2-9   epilogue: warps 2-5 drain token rows 0-127 (accumulator 0), warps 6-9 rows 128-255
// Every mbarrier wait is bounded (ptx.cuh).
#include "common.cuh"
#include "gemm_common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace w8a8 {
namespace {

constexpr int BLOCK_M = 256;
constexpr int BLOCK_N = 256;
constexpr int BLOCK_K = 128;
constexpr int UMMA_K = 32;
constexpr int STAGES = 3;
constexpr int A_HALF = 128 * BLOCK_K;          // one 128-row box of activations
constexpr int A_BYTES = 2 * A_HALF;
constexpr int B_BYTES = BLOCK_N * BLOCK_K;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 64 KiB
constexpr int TMEM_COLS = 512;
constexpr int kThreads = 320;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

template <class T, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmDev p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    uint8_t *gen_tiles = smem_raw + (tiles - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen_tiles + STAGES * STAGE_BYTES);
    const uint32_t bar_base = tiles + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t accf_bar = bar_base + 8u * (2 * STAGES);
    const uint32_t acce_bar = bar_base + 8u * (2 * STAGES + 1);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 2);
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
        mbar_init(accf_bar, 1);
        mbar_init(acce_bar, 8);  // one arrival per epilogue warp
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
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, WAIT_STAGE_EMPTY))) break;
                    mbar_expect_tx(full_bar(stage), STAGE_BYTES);
                    const uint32_t dst = tiles + stage * STAGE_BYTES;
                    tma_load_2d(dst, &map_a, kb * BLOCK_K, m_blk * BLOCK_M, full_bar(stage));
                    tma_load_2d(dst + A_HALF, &map_a, kb * BLOCK_K, m_blk * BLOCK_M + 128, full_bar(stage));
                    tma_load_2d(dst + A_BYTES, &map_b, kb * BLOCK_K, n_blk * BLOCK_N, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                for (int s = 0; s < STAGES; ++s) {
                    const unsigned long long t0 = global_ns();
                    const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
                    while (!mbar_try_wait(full_bar(s), par) && global_ns() - t0 < kWaitLimitNs / 4) {}
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(128, BLOCK_N);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                // both accumulators must have been drained by the epilogue of the previous tile
                if (!(ok = mbar_wait(acce_bar, ((uint32_t)it & 1u) ^ 1u, abort_flag, p.status, WAIT_ACC_EMPTY))) break;
                tc_fence_after();
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, p.status, WAIT_TMA_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = tiles + stage * STAGE_BYTES;
                    const uint64_t a0_desc = smem_desc_sw128(a_addr);
                    const uint64_t a1_desc = smem_desc_sw128(a_addr + A_HALF);
                    const uint64_t b_desc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t koff = (uint64_t)((k * UMMA_K) >> 4);
                        const uint32_t accumulate = (kb | k) != 0 ? 1u : 0u;
                        umma_i8(tmem_base, a0_desc + koff, b_desc + koff, idesc, accumulate);
                        umma_i8(tmem_base + (uint32_t)BLOCK_N, a1_desc + koff, b_desc + koff, idesc, accumulate);
                    }
                    umma_commit(empty_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(accf_bar);
            }
        }
    } else {
        // epilogue warps 2..9: TMEM lane quarter = warp % 4; warps 2-5 take accumulator 0, warps 6-9 accumulator 1
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
            const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
            ok = mbar_wait(accf_bar, (uint32_t)it & 1u, abort_flag, p.status, WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int m = m_blk * BLOCK_M + half * 128 + quarter * 32 + lane;
            const bool m_ok = m < p.M;
            const float as = (EPI != EPI_ACC && m_ok) ? p.a_scale[m] : 0.0f;
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * BLOCK_N);
            drain_accumulator<T, EPI>(p, t_row, m, m_ok, as, n_blk * BLOCK_N, BLOCK_N);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <class T, int EPI> cudaError_t launch_inst(const CUtensorMap &ma, const CUtensorMap &mb, const GemmDev &d, cudaStream_t s) {
    const int tiles = ((d.M + BLOCK_M - 1) / BLOCK_M) * ((d.N + BLOCK_N - 1) / BLOCK_N);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    return launch_kernel(gemm_tcgen05_wide_kernel<T, EPI>, dim3(grid), dim3(kThreads), (size_t)SMEM_BYTES, s, ma, mb, d);
}
template <class T> cudaError_t launch_epi(int epi, const CUtensorMap &ma, const CUtensorMap &mb, const GemmDev &d, cudaStream_t s) {
    switch (epi) {
        case EPI_PLAIN: return launch_inst<T, EPI_PLAIN>(ma, mb, d, s);
        case EPI_RESIDUAL: return launch_inst<T, EPI_RESIDUAL>(ma, mb, d, s);
        case EPI_ACC: return launch_inst<T, EPI_ACC>(ma, mb, d, s);
        default: return cudaErrorInvalidValue;
    }
}
template <class T, int EPI> cudaError_t set_attr() {
    return cudaFuncSetAttribute(gemm_tcgen05_wide_kernel<T, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
}

}  // namespace

cudaError_t init_gemm_tcgen05_wide() {
    cudaError_t e;
    if ((e = set_attr<Bf16, EPI_PLAIN>()) != cudaSuccess) return e;
    if ((e = set_attr<Bf16, EPI_RESIDUAL>()) != cudaSuccess) return e;
    if ((e = set_attr<Bf16, EPI_ACC>()) != cudaSuccess) return e;
    if ((e = set_attr<F32, EPI_PLAIN>()) != cudaSuccess) return e;
    if ((e = set_attr<F32, EPI_RESIDUAL>()) != cudaSuccess) return e;
    if ((e = set_attr<F32, EPI_ACC>()) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t launch_gemm_tcgen05_wide(const LinearArgs &l, const w8a8_weight *wt, cudaStream_t s) {
    if (!wt || !wt->has_maps || l.count != 1) return cudaErrorInvalidValue;
    CUtensorMap map_a;  // box of 128 token rows; a 256-row tile takes two
    cudaError_t e = encode_tile_map(&map_a, l.q, l.M, l.K, 128);
    if (e != cudaSuccess) return e;
    GemmDev d{};
    d.a_scale = l.a_scale; d.w_scale = wt->w_scale; d.M = l.M; d.N = wt->N; d.K = l.K;
    d.y = l.out[0]; d.residual = l.residual; d.combined = l.combined; d.acc = l.acc;
    d.status = device_status_ptr();
    return l.dtype == 0 ? launch_epi<Bf16>(l.epilogue, map_a, wt->map_rows256, d, s)
                        : launch_epi<F32>(l.epilogue, map_a, wt->map_rows256, d, s);
}

}  // namespace w8a8
