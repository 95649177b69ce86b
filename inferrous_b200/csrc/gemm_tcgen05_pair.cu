// Prefill-regime W8A8 projection on CTA pairs (sm_100a): tcgen05.mma.cta_group::2 computes a
// 256x256 output tile across two SMs.  Each CTA of the pair stages only its own half of both
// operands (128 token rows and 128 weight rows per 128-byte K block) and keeps two 256-column
// accumulators for its 128 token rows, so compared with the single-CTA 128x256 tile the operand
// traffic from L2 per multiply drops by a third while the epilogue still overlaps the next tile.
//
// Replaces the same reference kernels as gemm_tcgen05.cu (linear_large, src/kernels.rs:1145-1289).
// Roles per CTA (192 threads):
//   warp 0      TMA producer: 6-stage ring of {A half 128x128 B, B half 128x128 B}; the copies of BOTH
//               CTAs report their bytes to the leader CTA's "full" barrier (no cluster multicast:
//               every CTA loads only its own tiles)
//   warp 1      leader CTA only: one lane issues 4 x tcgen05.mma.cta_group::2 (M256 N256 K32) per stage
//               and commits to the "empty" / "accumulator full" barriers of both CTAs; in both CTAs
//               this warp owns the pair-wide tensor-memory allocation
//   warps 2-5   epilogue of the CTA's own 128 rows; hand the accumulator back by arriving on the
//               leader's "accumulator empty" barrier
// Every mbarrier wait is bounded (ptx.cuh); the two CTAs meet at cluster barriers after set-up and before exit.
#include "common.cuh"
#include "gemm_common.cuh"
#include "internal.h"
#include "ptx.cuh"

#include <cstdlib>

namespace w8a8 {
namespace {

constexpr int TILE_M = 256;
constexpr int BLOCK_K = 128, UMMA_K = 32;
constexpr int HALF_BYTES = 128 * BLOCK_K;       // this CTA's half of the token rows: one 128-row box
constexpr int TMEM_COLS = 512;
constexpr int kThreads = 192;
// Output channels per tile: 256, 192 or 128 (each CTA stages half of them).  The narrower tiles exist for the shapes
// whose 256-channel tiles leave the last wave over the 74 CTA pairs mostly empty (Q|K|V at 4096 tokens: 384 tiles = 5.2
// waves; with 192 channels 512 tiles = 6.9 waves).
template <int BN> struct PairTile {
    static constexpr int kHalfB = (BN / 2) * BLOCK_K;                 // this CTA's half of the weight rows
    static constexpr int kStageBytes = HALF_BYTES + kHalfB;
    static constexpr int kStages = (196 * 1024) / kStageBytes;        // 6, 7, 8
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in the CTA of rank `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tile copy whose byte count is reported to the barrier at the same offset in the pair's leader CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive, once the MMAs issued so far are complete, on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask)
                 : "memory");
}

template <class T, int EPI, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmDev p) {
    constexpr int TILE_N = BN, STAGES = PairTile<BN>::kStages, STAGE_BYTES = PairTile<BN>::kStageBytes;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    uint8_t *gen_tiles = smem_raw + (tiles - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen_tiles + STAGES * STAGE_BYTES);
    const uint32_t bar_base = tiles + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                 // used in the leader
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };     // one per CTA
    auto accf_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };  // one per CTA
    auto acce_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };  // used in the leader
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int m_tiles = (p.M + TILE_M - 1) / TILE_M;
    const int n_tiles = (p.N + TILE_N - 1) / TILE_N;
    const int num_tiles = m_tiles * n_tiles;
    const int num_kb = p.K / BLOCK_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);   // the leader's arrive.expect_tx; bytes of both CTAs complete it
            mbar_init(empty_bar(s), 1);  // the leader's multicast commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(accf_bar(a), 1);   // the leader's multicast commit
            mbar_init(acce_bar(a), 8);   // 4 epilogue warps x 2 CTAs (leader's copy is the one in use)
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anybody signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    dependency_wait();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs): own halves of A and B ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
                const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, WAIT_STAGE_EMPTY))) break;
                    const uint32_t leader_full = map_to_rank(full_bar(stage), 0);  // same offset in the leader CTA
                    if (leader) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
                    const uint32_t dst = tiles + stage * STAGE_BYTES;
                    tma_load_2d_pair(dst, &map_a, kb * BLOCK_K, m_blk * TILE_M + (int)rank * 128, leader_full);
                    tma_load_2d_pair(dst + HALF_BYTES, &map_b, kb * BLOCK_K, n_blk * TILE_N + (int)rank * (TILE_N / 2), leader_full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok && leader) {
                // Abandoned: the leader's "full" barriers count the bytes of both CTAs, so once they have
                // completed (bounded wait) no copy of the pair is in flight; the peer stays until the final
                // cluster barrier, which the leader reaches only after this.
                for (int s = 0; s < STAGES; ++s) {
                    const unsigned long long t0 = global_ns();
                    const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
                    while (!mbar_try_wait(full_bar(s), par) && global_ns() - t0 < kWaitLimitNs / 4) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (leader && lane == 0) {
            constexpr uint32_t idesc = make_idesc(TILE_M, TILE_N);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!(ok = mbar_wait(acce_bar(acc), acc_phase ^ 1u, abort_flag, p.status, WAIT_ACC_EMPTY))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * TILE_N);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, p.status, WAIT_TMA_FULL))) break;
                    tc_fence_after();
                    const uint32_t a_addr = tiles + stage * STAGE_BYTES;
                    const uint64_t a_desc = smem_desc_sw128(a_addr);
                    const uint64_t b_desc = smem_desc_sw128(a_addr + HALF_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t koff = (uint64_t)((k * UMMA_K) >> 4);
                        umma_i8_pair(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(empty_bar(stage));  // both CTAs may refill this stage
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit_pair(accf_bar(acc));  // both CTAs may drain this accumulator
            }
        }
    } else {
        // ---------------- epilogue warps (both CTAs): own 128 token rows, all 256 columns ----------------
        const int quarter = warp & 3;
        int it = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++it) {
            const int m_blk = tile % m_tiles, n_blk = tile / m_tiles;
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            ok = mbar_wait(accf_bar(acc), acc_phase, abort_flag, p.status, WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int m = m_blk * TILE_M + (int)rank * 128 + quarter * 32 + lane;
            const bool m_ok = m < p.M;
            const float as = (EPI != EPI_ACC && m_ok) ? p.a_scale[m] : 0.0f;
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * TILE_N);
            drain_accumulator<T, EPI>(p, t_row, m, m_ok, as, n_blk * TILE_N, TILE_N);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(acce_bar(acc), 0));
        }
    }

    // common exit: nobody leaves while the peer may still signal or read this CTA's shared memory
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

template <class T, int EPI, int BN> cudaError_t launch_inst(const CUtensorMap &ma, const CUtensorMap &mb, const GemmDev &d, cudaStream_t s) {
    const int tiles = ((d.M + TILE_M - 1) / TILE_M) * ((d.N + BN - 1) / BN);
    int pairs = sm_count() / 2;
    if (tiles < pairs) pairs = tiles;
    return launch_kernel(gemm_tcgen05_pair_kernel<T, EPI, BN>, dim3(2 * pairs), dim3(kThreads), (size_t)PairTile<BN>::kSmemBytes, s, ma, mb, d);
}
template <class T, int BN> cudaError_t launch_epi(int epi, const CUtensorMap &ma, const CUtensorMap &mb, const GemmDev &d, cudaStream_t s) {
    switch (epi) {
        case EPI_PLAIN: return launch_inst<T, EPI_PLAIN, BN>(ma, mb, d, s);
        case EPI_RESIDUAL: return launch_inst<T, EPI_RESIDUAL, BN>(ma, mb, d, s);
        case EPI_ACC: return launch_inst<T, EPI_ACC, BN>(ma, mb, d, s);
        default: return cudaErrorInvalidValue;
    }
}
template <class T, int BN> cudaError_t set_attrs() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<T, EPI_PLAIN, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairTile<BN>::kSmemBytes))) return e;
    if ((e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<T, EPI_RESIDUAL, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairTile<BN>::kSmemBytes))) return e;
    return cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<T, EPI_ACC, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairTile<BN>::kSmemBytes);
}

// Channels per tile: the width with the least (waves over the CTA pairs) x (time of one tile, measured to go as
// BN + 64: a 192-channel tile takes 0.80 of a 256-channel one); the wider one on a tie.  Measured at 4096 tokens:
// Q|K|V 96.1 -> 90.1 us with 192 channels (6 -> 7 waves of smaller tiles); O, down, gate|up stay at 256; 128-channel
// tiles lost everywhere (their K loop is bound by the token rows staged per block) and exist for tests.
}  // namespace

int pair_tile_channels(int M, int N) {
    if (const char *force = getenv("W8A8_PAIR_BN")) {
        const int bn = atoi(force);
        if (bn == 256 || bn == 192 || bn == 128) return bn;
    }
    const long long pairs = sm_count() / 2, m_tiles = (M + TILE_M - 1) / TILE_M;
    int best = 256;
    long long best_cost = -1;
    for (int bn : {256, 192}) {
        const long long tiles = m_tiles * ((N + bn - 1) / bn);
        const long long cost = ((tiles + pairs - 1) / pairs) * (bn + 64);
        if (best_cost < 0 || cost < best_cost) {
            best = bn;
            best_cost = cost;
        }
    }
    return best;
}

cudaError_t init_gemm_tcgen05_pair() {
    cudaError_t e;
    if ((e = set_attrs<Bf16, 256>()) != cudaSuccess) return e;
    if ((e = set_attrs<Bf16, 192>()) != cudaSuccess) return e;
    if ((e = set_attrs<Bf16, 128>()) != cudaSuccess) return e;
    if ((e = set_attrs<F32, 256>()) != cudaSuccess) return e;
    if ((e = set_attrs<F32, 192>()) != cudaSuccess) return e;
    return set_attrs<F32, 128>();
}

cudaError_t launch_gemm_tcgen05_pair(const LinearArgs &l, const w8a8_weight *wt, cudaStream_t s) {
    if (!wt || !wt->has_maps || l.count != 1) return cudaErrorInvalidValue;
    CUtensorMap map_a;
    cudaError_t e = encode_tile_map(&map_a, l.q, l.M, l.K, 128);
    if (e != cudaSuccess) return e;
    GemmDev d{};
    d.a_scale = l.a_scale; d.w_scale = wt->w_scale; d.M = l.M; d.N = wt->N; d.K = l.K;
    d.y = l.out[0]; d.residual = l.residual; d.combined = l.combined; d.acc = l.acc;
    d.status = device_status_ptr();
    switch (pair_tile_channels(l.M, wt->N)) {
        case 192:
            return l.dtype == 0 ? launch_epi<Bf16, 192>(l.epilogue, map_a, wt->map_rows96, d, s)
                                : launch_epi<F32, 192>(l.epilogue, map_a, wt->map_rows96, d, s);
        case 128:
            return l.dtype == 0 ? launch_epi<Bf16, 128>(l.epilogue, map_a, wt->map_rows64, d, s)
                                : launch_epi<F32, 128>(l.epilogue, map_a, wt->map_rows64, d, s);
        default:
            return l.dtype == 0 ? launch_epi<Bf16, 256>(l.epilogue, map_a, wt->map_rows128, d, s)
                                : launch_epi<F32, 256>(l.epilogue, map_a, wt->map_rows128, d, s);
    }
}

}  // namespace w8a8
