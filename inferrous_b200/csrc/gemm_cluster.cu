// W8A8 projection for 9..256 tokens against the small and mid-sized matrices (Q|K|V, O, down: 16-50 MB), where the
// product is bound by one pass over the int8 weights and by fixed latencies, and where a tile per SM would leave most
// of the GPU idle (N = 4096 is 32 tiles of 128 channels).
//
// Replaces, from crates/inferrous-qwen3/src/kernels.rs: linear_splitk (:935-1034, 2..31 rows) and linear_tiled
// (:1038-1141, 32..255 rows) with their host dispatch (src/gpu.rs:473-494).  The reference splits K over the eight warps
// of a CTA and reduces through shared memory.  Here K is split over the CTAs of a thread-block cluster and the int32
// partial sums meet in DISTRIBUTED shared memory, so no global scratch, atomics or arrival counters are involved:
//   * one cluster of S CTAs (S = 1, 2, 4 or 8, chosen so that tiles x S fills the SMs) per tile of 128 output channels;
//     CTA r of the cluster owns the r-th share of the K blocks;
//   * per CTA: warp 0 = TMA producer (weight box 128 x 128 B, token box NTOK x 128 B, 128-byte swizzle, a ring of
//     stages), warp 1 = one lane issuing tcgen05.mma.cta_group::1.kind::i8 M128 x N(NTOK) x K32 with the WEIGHTS on
//     the MMA's M side (swap-AB: no MMA rows are spent on absent tokens) into tensor memory, warps 2-5 = epilogue;
//   * after its K share every CTA spills its accumulator (lane = channel, column = token) to its own shared memory as
//     [token][channel] int32, the cluster meets at a hardware barrier, and CTA r sums the S partials of ITS 128 / S
//     channels straight out of the peers' shared memory (ld.shared::cluster), dequantizes and stores -- a
//     reduce-scatter inside the cluster; a second cluster barrier keeps every CTA's memory alive until all have read.
// int32 addition is exact, so the result is bit-identical to every other variant.  Every mbarrier wait is bounded
// (ptx.cuh); a CTA whose wait ran out still arrives at both cluster barriers and stores nothing.
#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"

#include <algorithm>

namespace w8a8 {
namespace {

constexpr int TILE_N = 128;   // output channels per tile (UMMA M)
constexpr int BLOCK_K = 128;  // bytes of K per block
constexpr int UMMA_K = 32;
constexpr int A_BYTES = TILE_N * BLOCK_K;
constexpr int kThreads = 192;
constexpr int kSmemBudget = 200 * 1024;
constexpr int kMaxTokens = 256;

struct ClusterDev {
    const float *a_scale;
    const float *w_scale;
    int M, N, K, ntok;  // ntok = tokens padded to a multiple of 16
    int stages, split;  // ring depth; CTAs per cluster
    void *y;
    const void *residual;
    void *combined;
    int32_t *acc;
    uint32_t *status;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_smem(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ int4 ld_cluster_16(uint32_t addr) {
    int4 v;
    asm volatile("ld.shared::cluster.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

template <class T, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_cluster_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q, const ClusterDev p) {
    typedef typename T::storage S;
    extern __shared__ uint8_t smem_raw[];
    const int NS = p.stages;
    const int b_bytes = p.ntok * BLOCK_K;
    const int stage_bytes = A_BYTES + b_bytes;  // multiple of 1024: ntok is a multiple of 16
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (tiles - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(gen + (size_t)NS * stage_bytes);
    const uint32_t bar_base = tiles + (uint32_t)(NS * stage_bytes);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (NS + s); };
    const uint32_t accf_bar = bar_base + 8u * (2 * NS);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * NS + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int32_t *part = reinterpret_cast<int32_t *>(gen);  // [ntok][128] partial sums, over the ring once the MMAs are done
    const uint32_t part_addr = tiles;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = p.split;
    const uint32_t rank = cluster_rank();
    const int tile = blockIdx.x / split;
    const int blocks = p.K / BLOCK_K;
    const int kb_begin = (int)((long long)rank * blocks / split), kb_end = (int)((long long)(rank + 1) * blocks / split);
    const int tmem_cols = p.ntok <= 32 ? 32 : (p.ntok <= 64 ? 64 : (p.ntok <= 128 ? 128 : 256));

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(accf_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), (uint32_t)tmem_cols);
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
        for (int kb = kb_begin; kb < kb_end && ok; ++kb) {
            if (lane == 0) ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, WAIT_STAGE_EMPTY);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane == 0) {
                mbar_expect_tx(full_bar(stage), (uint32_t)stage_bytes);
                const uint32_t dst = tiles + (uint32_t)(stage * stage_bytes);
                // weights are immutable: their copies may start before the predecessor kernel is done
                tma_load_2d(dst, &map_w, kb * BLOCK_K, tile * TILE_N, full_bar(stage));
                if (!waited) {
                    dependency_wait();
                    waited = true;
                }
                tma_load_2d(dst + (uint32_t)A_BYTES, &map_q, kb * BLOCK_K, 0, full_bar(stage));
            }
            if (++stage == NS) { stage = 0; phase ^= 1u; }
        }
        if (!ok && lane == 0) {  // abandoned: let the copies already issued land before the memory is reused or freed
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
            bool ok = true;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag, p.status, WAIT_TMA_FULL))) break;
                tc_fence_after();
                const uint32_t a_addr = tiles + (uint32_t)(stage * stage_bytes);
                const uint64_t a_desc = smem_desc_sw128(a_addr);
                const uint64_t b_desc = smem_desc_sw128(a_addr + (uint32_t)A_BYTES);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t koff = (uint64_t)((k * UMMA_K) >> 4);
                    umma_i8(tmem_base, a_desc + koff, b_desc + koff, idesc, (kb != kb_begin || k != 0) ? 1u : 0u);
                }
                umma_commit(empty_bar(stage));
                if (++stage == NS) { stage = 0; phase ^= 1u; }
            }
            if (ok) umma_commit(accf_bar);
        }
    } else {
        // ---------------- epilogue warps, first half: accumulator -> own shared memory ----------------
        dependency_wait();
        const int quarter = warp & 3;
        bool ok = mbar_wait(accf_bar, 0u, abort_flag, p.status, WAIT_ACC_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {  // every MMA has completed, so the ring is free: the partial tile goes on top of it
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
            for (int c0 = 0; c0 < p.ntok; c0 += 16) {
                int v[16];
                tmem_ld_32x16(t_row + (uint32_t)c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) part[(c0 + i) * TILE_N + quarter * 32 + lane] = v[i];
            }
        }
    }

    // ---- the cluster meets: every CTA's partial tile is in its shared memory (or the CTA gave up) ----
    tc_fence_before();
    __syncthreads();
    const bool mine_ok = *abort_flag == 0;
    cluster_barrier();

    if (warp >= 2 && mine_ok) {
        // ---------------- second half: CTA `rank` finishes channels [rank * 128 / split, (rank + 1) * 128 / split) ----------------
        const int width = TILE_N / split;          // 128, 64, 32 or 16 channels, in groups of 4
        const int groups = width / 4;
        const int t = threadIdx.x - 64;            // 0 .. 127
        const int n_base = tile * TILE_N + (int)rank * width;
        for (int idx = t; idx < p.M * groups; idx += 128) {
            const int m = idx / groups, c4 = (idx % groups) * 4;
            const int n = n_base + c4;
            if (n >= p.N) continue;
            const uint32_t off = part_addr + (uint32_t)((m * TILE_N + (int)rank * width + c4) * 4);
            int4 sum = make_int4(0, 0, 0, 0);
            for (int s = 0; s < split; ++s) {
                const int4 v = ld_cluster_16(peer_smem(off, (uint32_t)s));
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            const int acc[4] = {sum.x, sum.y, sum.z, sum.w};
            const int64_t o = (int64_t)m * p.N + n;
            if (EPI == EPI_ACC) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (n + i < p.N) p.acc[o + i] = acc[i];
                continue;
            }
            const float as = p.a_scale[m];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (n + i >= p.N) break;
                const float y = dequant(acc[i], as, p.w_scale[n + i]);
                if (p.y) T::store(static_cast<S *>(p.y) + o + i, y);
                if (EPI == EPI_RESIDUAL) {
                    const float r = T::load(static_cast<const S *>(p.residual) + o + i);
                    T::store(static_cast<S *>(p.combined) + o + i, bf16_rne(__fadd_rn(r, y)));
                }
            }
        }
    }

    // nobody leaves while a peer may still read this CTA's shared memory
    cluster_barrier();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)tmem_cols);
    }
}

template <class T, int EPI>
cudaError_t launch_inst(const CUtensorMap &mw, const CUtensorMap &mq, const ClusterDev &d, int grid, size_t smem, cudaStream_t s) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = (unsigned)d.split;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
    if (programmatic_launch_enabled()) {
        attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attrs;
    return cudaLaunchKernelEx(&cfg, gemm_cluster_kernel<T, EPI>, mw, mq, d);
}
template <class T>
cudaError_t launch_epi(int epi, const CUtensorMap &mw, const CUtensorMap &mq, const ClusterDev &d, int grid, size_t smem, cudaStream_t s) {
    switch (epi) {
        case EPI_PLAIN: return launch_inst<T, EPI_PLAIN>(mw, mq, d, grid, smem, s);
        case EPI_RESIDUAL: return launch_inst<T, EPI_RESIDUAL>(mw, mq, d, grid, smem, s);
        case EPI_ACC: return launch_inst<T, EPI_ACC>(mw, mq, d, grid, smem, s);
        default: return cudaErrorInvalidValue;
    }
}
template <class T, int EPI> cudaError_t set_attr() {
    return cudaFuncSetAttribute(gemm_cluster_kernel<T, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget + 2048);
}

}  // namespace

cudaError_t init_gemm_cluster() {
    cudaError_t e;
    if ((e = set_attr<Bf16, EPI_PLAIN>()) != cudaSuccess) return e;
    if ((e = set_attr<Bf16, EPI_RESIDUAL>()) != cudaSuccess) return e;
    if ((e = set_attr<Bf16, EPI_ACC>()) != cudaSuccess) return e;
    if ((e = set_attr<F32, EPI_PLAIN>()) != cudaSuccess) return e;
    if ((e = set_attr<F32, EPI_RESIDUAL>()) != cudaSuccess) return e;
    if ((e = set_attr<F32, EPI_ACC>()) != cudaSuccess) return e;
    return cudaSuccess;
}

// CTAs per cluster: the largest of 8, 4, 2, 1 for which every cluster of the launch is resident at once (tiles x S
// CTAs on the SMs) and every CTA still has at least two K blocks.
int cluster_split(int N, int K) {
    const int tiles = (N + TILE_N - 1) / TILE_N, blocks = K / BLOCK_K;
    int split = 8;
    while (split > 1 && (tiles * split > sm_count() || blocks / split < 2)) split /= 2;
    return split;
}

cudaError_t launch_gemm_cluster(const LinearArgs &l, const w8a8_weight *wt, cudaStream_t s) {
    if (!wt || !wt->has_maps || l.count != 1 || l.M < 1 || l.M > kMaxTokens || l.K < BLOCK_K) return cudaErrorInvalidValue;
    const int ntok = (l.M + 15) / 16 * 16;
    CUtensorMap map_q;
    cudaError_t e = encode_tile_map(&map_q, l.q, l.M, l.K, ntok);
    if (e != cudaSuccess) return e;
    ClusterDev d{};
    d.a_scale = l.a_scale; d.w_scale = wt->w_scale; d.M = l.M; d.N = wt->N; d.K = l.K; d.ntok = ntok;
    d.split = cluster_split(wt->N, l.K);
    const int stage_bytes = A_BYTES + ntok * BLOCK_K;
    const int share = (l.K / BLOCK_K + d.split - 1) / d.split;  // K blocks of the busiest CTA
    d.stages = std::max(2, std::min(std::min(8, share), (kSmemBudget - 1024) / stage_bytes));
    // the partial tile ([ntok][128] int32) is spilled on top of the ring: the ring must be at least that large
    d.stages = std::max(d.stages, (ntok * TILE_N * 4 + stage_bytes - 1) / stage_bytes);
    d.y = l.out[0]; d.residual = l.residual; d.combined = l.combined; d.acc = l.acc;
    d.status = device_status_ptr();
    const int grid = ((wt->N + TILE_N - 1) / TILE_N) * d.split;
    const size_t smem = (size_t)d.stages * stage_bytes + 1024 + 8 * (2 * (size_t)d.stages + 1) + 64;
    return l.dtype == 0 ? launch_epi<Bf16>(l.epilogue, wt->map_rows128, map_q, d, grid, smem, s)
                        : launch_epi<F32>(l.epilogue, wt->map_rows128, map_q, d, grid, smem, s);
}

}  // namespace w8a8
