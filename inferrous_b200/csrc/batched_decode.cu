// Batched ("ragged") decode: one new token for each of `rows` independent sequences, every sequence with its own
// position and its own KV cache, plus greedy selection on stored logits for batches that the fused head + selection
// kernel does not cover.
//
// The reference serves one request at a time (crates/inferrous-qwen3/src/gpu.rs:818-929; replicas and batching are
// deferred, docs/plans/production.md:87); its attention kernel computes, per (row, head),
//   out = softmax(q . K[0 .. position] * 128^-0.5) . V[0 .. position]            (src/kernels.rs:1490-1658)
// and that function is what attention_batched_kernel computes for every row against that row's own cache.  What is
// new is the launch shape only:
//   * one CTA serves the GH query heads that share a key/value head (grouped-query attention): every key and value
//     line is fetched once for the group instead of once per head -- in batched decode the KV cache, not the weights,
//     is the larger stream (64 sequences of 2 000 keys read 0.55 GB per layer against 0.19 GB of weights);
//   * the keys of a row are split into units of 512 (up to 8) whose partial (maximum, total, sums) the last CTA to
//     arrive combines, so a short and a long sequence in the same batch both spread over the GPU.  The units are a
//     function of the row's context length alone, never of the batch: a sequence decoded alone and the same sequence
//     decoded inside a batch produce the same bits;
//   * both products run on the tensor cores (warp-level bf16 MMA, float32 accumulation) with the keys, not the query
//     rows, on the MMA's 16-row side; the kernel is bound by the stream of keys and values from HBM.
// float32 sums are reassociated relative to the reference's one-thread-per-key kernel (q, k, v are bf16 values, so every
// product is exact and only the additions round; the softmax weights are carried as two bf16 parts); the result stays
// inside the reference's own bound for this operator (|err| <= 2e-4 + 1 % |x|, docs/qwen3-8b-w8a8/coverage.md:28).
// The legacy warp-level MMA is deliberate: a tile of 32 keys x 4 heads per warp is far below tcgen05's 128-row
// granularity, and attention is not on the W8A8 path.
#include "../../include/qwen3_glue.h"
#include "../../include/w8a8.h"
#include "common.cuh"
#include "internal.h"

#include <algorithm>

namespace w8a8 {
namespace {

constexpr int kHeadDim = 128;
constexpr int kMaxContext = 4096;     // src/lib.rs:18
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kStepKeys = 32;         // keys a warp stages and multiplies at a time
constexpr int kWarpKeys = 128;        // consecutive keys per warp and item
constexpr int kUnitKeys = kWarps * kWarpKeys;         // keys per item: 512
constexpr int kMaxUnits = kMaxContext / kUnitKeys;    // 8 items for the longest context
constexpr int kPitch = kHeadDim + 8;  // bf16 elements per staged row: 272 bytes, conflict-free for ldmatrix
constexpr size_t kSmemBytes = (size_t)2 * kWarps * kStepKeys * kPitch * sizeof(uint16_t);  // keys + values: 68 KiB, three CTAs per SM
constexpr int kRecord = kHeadDim + 4;  // floats per (row, head, split) in the workspace: 128 sums, maximum, total, padding

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void record_range_fault(uint32_t *status, uint32_t detail) {
    if (status && atomicCAS(status, 0u, (uint32_t)FAULT_CACHE_RANGE) == 0u) status[1] = detail;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {  // both already bf16-representable
    return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xffff0000u);
}
// The transpose of an 8 x 8 matrix of 16-bit elements held one 32-bit register per lane (row = lane / 4, two columns).
__device__ __forceinline__ uint32_t transpose_8x8(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// A fixed number of CTAs (as many as the GPU holds at once, three per SM) of four warps each work through the launch's
// items -- one item per (row, unit of 512 keys, group of GH query heads that share a key/value head), found from the
// rows' positions by a prefix sum that every CTA computes for itself and handed out through a ticket counter, so rows
// with short contexts cost nothing and the launch shape never depends on the positions (a captured graph replays for any
// of them).  Within an item every warp is an independent pipeline over its own 128 consecutive keys, 32 at a time:
//   stage    32 key rows, then 32 value rows, go to the warp's part of shared memory with 16-byte asynchronous copies;
//            the next step's keys are requested as soon as the scores of this step are computed and its values as soon
//            as the second product is done, so copies and arithmetic overlap inside every warp (up to 192 KiB in flight
//            per SM)
//   scores   S^T = K . Q^T on mma.sync.m16n8k16 (bf16 x bf16 -> f32): the keys are the MMA's 16 rows, the GH query heads
//            its 8 columns, so no tensor-core work is spent on absent rows; score = dot * 128^-0.5
//   softmax  running maximum and total per head (flash attention): e = exp(score - maximum) in the reference's
//            ex2.approx form, earlier sums rescaled by exp(old maximum - new maximum)
//   P.V      O^T += V^T . P^T on the same MMA: the value tile is read through ldmatrix.trans, each float32 weight enters
//            as hi + lo, two bf16 numbers (hi = bf16(p), lo = bf16(p - hi)), moved from the accumulator layout of the
//            first product to the operand layout of the second with movmatrix
//   combine  (maximum, total, sums) of the four warps, then of the row's units by the last CTA to arrive, with weights
//            exp(m - M) -- flash decoding.  No CTA ever waits for another.
// The association depends on nothing but the row's context length.
constexpr int kMaxRows = 256;  // rows per launch (the prefix sum over the rows lives in shared memory); the entry point cuts larger batches

template <class T, int GH>
__global__ void __launch_bounds__(kThreads, 3) attention_batched_kernel(const typename T::storage *__restrict__ q, int64_t ldq, int rows,
                                                                        int q_heads, int kv_heads, const uint16_t *__restrict__ k_cache,
                                                                        const uint16_t *__restrict__ v_cache, int64_t cache_stride,
                                                                        const uint32_t *__restrict__ positions,
                                                                        typename T::storage *__restrict__ out, int64_t ldo, int capacity,
                                                                        uint32_t *maxima, float *scratch, uint32_t *counters,
                                                                        uint32_t *tickets, uint32_t *status) {
    extern __shared__ __align__(16) uint16_t tile_smem[];
    typedef uint16_t (*TilePtr)[kPitch];
    TilePtr ks = reinterpret_cast<TilePtr>(tile_smem);  // [4 warps][32 keys]
    TilePtr vs = ks + kWarps * kStepKeys;
    __shared__ float warp_max[kWarps][8], warp_total[kWarps][8];
    __shared__ float unit_weight[8][kMaxUnits], unit_den[8];
    __shared__ int first_unit[kMaxRows + 1];  // exclusive prefix sum of the rows' unit counts
    __shared__ int row_end[kMaxRows];         // visible keys per row
    __shared__ int scan_warp[kWarps];
    __shared__ uint32_t arrived, ticket[2];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31, g = lane >> 2, tq = lane & 3;
    const int group = q_heads / kv_heads, chunks = group / GH;
    const int groups = kv_heads * chunks;  // head groups per row

    // Work list: row r has ceil((positions[r] + 1) / 512) units (none if its position lies beyond the cache: the row is
    // skipped and reported).  The positions were uploaded by the host before the step began, so they do not depend on the
    // preceding kernel and all of this runs before the dependency wait.
    {
        constexpr int kPer = kMaxRows / kThreads;  // consecutive rows per thread
        int mine[kPer], total = 0;
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int r = t * kPer + i;
            int n = 0;
            if (r < rows) {
                const uint32_t end_u = positions[r] + 1u;
                if (end_u > (uint32_t)capacity) {
                    if (blockIdx.x == 0) record_range_fault(status, end_u);
                    row_end[r] = 0;
                } else {
                    n = ((int)end_u + kUnitKeys - 1) / kUnitKeys;
                    row_end[r] = (int)end_u;
                }
            }
            mine[i] = total;
            total += n;
        }
        int incl = total;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        if (lane == 31) scan_warp[warp] = incl;
        __syncthreads();
        int base = incl - total;
        for (int w = 0; w < warp; ++w) base += scan_warp[w];
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int r = t * kPer + i;
            if (r < rows) first_unit[r] = base + mine[i];
        }
        if (t == kThreads - 1) first_unit[rows] = base + total;  // rows beyond `rows` contributed nothing
        __syncthreads();
    }
    const uint32_t items = (uint32_t)first_unit[rows] * (uint32_t)groups;
    const size_t key_stride = (size_t)kv_heads * kHeadDim;
    const int r0 = warp * kStepKeys;  // this warp's rows of the two tiles
    float *mine_o = reinterpret_cast<float *>(&ks[r0][0]);  // [GH][128] partial sums, over this warp's key rows once read
    const int part = lane & 15, half = lane >> 4;

    // Items are handed out through a ticket counter (tickets[0]; zero between launches), so a CTA that starts late or
    // runs on a slower SM simply takes fewer; which CTA computes an item has no influence on the result.  The counter
    // belongs to this launch only after the preceding kernels have finished, hence after the dependency wait.  The next
    // ticket is drawn while the current item is being worked on.
    dependency_wait();
    if (t == 0) ticket[0] = atomicAdd(tickets, 1u);
    __syncthreads();
    for (int turn = 0;; turn ^= 1) {
        const uint32_t item = ticket[turn];
        if (item >= items) break;
        if (t == 0) ticket[turn ^ 1] = atomicAdd(tickets, 1u);  // read after the barrier that ends this item
        const int ju = (int)(item / (uint32_t)groups), kvg = (int)(item % (uint32_t)groups);
        int row;
        {  // the row whose range of units holds ju: the last r with first_unit[r] <= ju
            int lo = 0, hi = rows;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (first_unit[mid] <= ju) lo = mid; else hi = mid;
            }
            row = lo;
        }
        const int unit = ju - first_unit[row];
        const int units = first_unit[row + 1] - first_unit[row];
        const int kv = kvg / chunks, head0 = kv * group + (kvg % chunks) * GH;
        const int end = row_end[row];
        const int wbegin = unit * kUnitKeys + warp * kWarpKeys;             // this warp's first key
        const int wcount = max(0, min(kWarpKeys, end - wbegin));            // and how many it has: 0 .. 128
        const int nsteps = (wcount + kStepKeys - 1) / kStepKeys;
        const uint16_t *kc = k_cache + (size_t)row * cache_stride + (size_t)kv * kHeadDim + (size_t)wbegin * key_stride + 8 * part;
        const uint16_t *vc = v_cache + (size_t)row * cache_stride + (size_t)kv * kHeadDim + (size_t)wbegin * key_stride + 8 * part;

        // 16 chunks of 16 bytes per row: a half-warp copies one row, the warp two rows per instruction
        auto stage = [&](TilePtr tile, const uint16_t *src, int step) {
            const uint16_t *p = src + (size_t)(step * kStepKeys + half) * key_stride;
#pragma unroll 4
            for (int i = 0; i < 16; ++i) {
                const int r = 2 * i + half;
                if (step * kStepKeys + r < wcount)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&tile[r0 + r][8 * part])), "l"(p));
                else  // rows past the end: zeros, so that 0 * value stays 0 in the second product
                    *reinterpret_cast<uint4 *>(&tile[r0 + r][8 * part]) = make_uint4(0, 0, 0, 0);
                p += 2 * key_stride;
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        float m_w[2] = {-INFINITY, -INFINITY}, l_w[2] = {0.0f, 0.0f};  // this lane's two heads: 2 tq and 2 tq + 1
        if (nsteps > 0) {
            stage(ks, kc, 0);
            stage(vs, vc, 0);
            // Q^T as the B operand: lane g holds head g (zeros beyond GH), 16 channels per step
            uint32_t qf[8][2];
            {
                const typename T::storage *qr = q + (size_t)row * ldq + (size_t)(head0 + (g < GH ? g : 0)) * kHeadDim + 2 * tq;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    qf[s][0] = g < GH ? pack_bf16(T::load(qr + 16 * s), T::load(qr + 16 * s + 1)) : 0u;
                    qf[s][1] = g < GH ? pack_bf16(T::load(qr + 16 * s + 8), T::load(qr + 16 * s + 9)) : 0u;
                }
            }
            float o[8][4];  // channels 16 dt + {g, g + 8} x heads {2 tq, 2 tq + 1}, unnormalised
#pragma unroll
            for (int dt = 0; dt < 8; ++dt)
#pragma unroll
                for (int i = 0; i < 4; ++i) o[dt][i] = 0.0f;
            const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
            const int v_row = (lane & 7) + 8 * (lane >> 4), v_col = 8 * ((lane >> 3) & 1);

            for (int step = 0; step < nsteps; ++step) {
                // copies are committed in the order K0 V0 K1 V1 ...: one group may stay in flight behind the one needed
                asm volatile("cp.async.wait_group 1;" ::: "memory");
                __syncwarp();
                // scores of 32 keys x GH heads, transposed: sc[mt] = keys 16 mt + {g, g + 8} x heads {2 tq, 2 tq + 1}
                float sc[2][4];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) sc[mt][i] = 0.0f;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        uint32_t a[4];
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                                     : "r"(smem_addr(&ks[r0 + 16 * mt + a_row][16 * s + a_col])));
                        mma_bf16(sc[mt], a, qf[s][0], qf[s][1]);
                    }
                }
                __syncwarp();  // the key rows are read
                if (step + 1 < nsteps)
                    stage(ks, kc, step + 1);
                else
                    asm volatile("cp.async.commit_group;" ::: "memory");  // keeps the group count in step
                // scale, mask, running maximum per head
                float m_new[2] = {m_w[0], m_w[1]};
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int key = step * kStepKeys + 16 * mt + g + 8 * (i >> 1), head = 2 * tq + (i & 1);
                        sc[mt][i] = (key < wcount && head < GH) ? __fmul_rn(sc[mt][i], 0.08838834764831845f) : -INFINITY;
                        m_new[i & 1] = fmaxf(m_new[i & 1], sc[mt][i]);
                    }
                float corr[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 4));
                    m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 8));
                    m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 16));
                    corr[e] = m_w[e] == -INFINITY ? 0.0f : exp_approx(__fadd_rn(m_w[e], -m_new[e]));  // nothing summed yet: 0
                    l_w[e] = __fmul_rn(l_w[e], corr[e]);
                    m_w[e] = m_new[e];
                }
#pragma unroll
                for (int dt = 0; dt < 8; ++dt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[dt][i] = __fmul_rn(o[dt][i], corr[i & 1]);
                // weights (hi + lo) in the operand layout of the second product, and their totals (per lane for now)
                uint32_t ph[2][2], pl[2][2];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    float hi[4], lo[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float base = m_w[i & 1];
                        const float p = base == -INFINITY ? 0.0f : exp_approx(__fadd_rn(sc[mt][i], -base));  // a masked score gives 0
                        l_w[i & 1] = __fadd_rn(l_w[i & 1], p);
                        hi[i] = bf16_rne(p);
                        lo[i] = bf16_rne(__fadd_rn(p, -hi[i]));
                    }
                    ph[mt][0] = transpose_8x8(pack_bf16(hi[0], hi[1]));
                    ph[mt][1] = transpose_8x8(pack_bf16(hi[2], hi[3]));
                    pl[mt][0] = transpose_8x8(pack_bf16(lo[0], lo[1]));
                    pl[mt][1] = transpose_8x8(pack_bf16(lo[2], lo[3]));
                }
                asm volatile("cp.async.wait_group 1;" ::: "memory");  // this step's values (the next keys may be in flight)
                __syncwarp();
                // O^T += V^T . P^T: eight tiles of 16 channels, two steps of 16 keys
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
                    for (int dt = 0; dt < 8; ++dt) {
                        uint32_t a[4];
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                                     : "r"(smem_addr(&vs[r0 + 16 * mt + v_row][16 * dt + v_col])));
                        mma_bf16(o[dt], a, ph[mt][0], ph[mt][1]);
                        mma_bf16(o[dt], a, pl[mt][0], pl[mt][1]);
                    }
                }
                __syncwarp();  // the value rows are read
                if (step + 1 < nsteps)
                    stage(vs, vc, step + 1);
                else
                    asm volatile("cp.async.commit_group;" ::: "memory");
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");  // only empty groups are left
#pragma unroll
            for (int e = 0; e < 2; ++e) {  // the lanes that share a head hold partial totals
                l_w[e] = __fadd_rn(l_w[e], __shfl_xor_sync(0xffffffffu, l_w[e], 4));
                l_w[e] = __fadd_rn(l_w[e], __shfl_xor_sync(0xffffffffu, l_w[e], 8));
                l_w[e] = __fadd_rn(l_w[e], __shfl_xor_sync(0xffffffffu, l_w[e], 16));
            }
#pragma unroll
            for (int dt = 0; dt < 8; ++dt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int head = 2 * tq + (i & 1);
                    if (head < GH) mine_o[head * kHeadDim + 16 * dt + g + 8 * (i >> 1)] = o[dt][i];
                }
        }
        if (g == 0) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                warp_max[warp][2 * tq + e] = m_w[e];
                warp_total[warp][2 * tq + e] = l_w[e];
            }
        }
        __syncthreads();

        // the four warps' partial results, thread = channel
        float sums[GH], tops[GH], dens[GH];
#pragma unroll
        for (int h = 0; h < GH; ++h) {
            float top = warp_max[0][h];
#pragma unroll
            for (int w = 1; w < kWarps; ++w) top = fmaxf(top, warp_max[w][h]);
            float sum = 0.0f, den = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float mw = warp_max[w][h];
                if (mw != -INFINITY) {  // a warp without keys left nothing behind
                    const float weight = exp_approx(__fadd_rn(mw, -top));
                    den = __fmaf_rn(warp_total[w][h], weight, den);
                    sum = __fmaf_rn(reinterpret_cast<const float *>(&ks[kStepKeys * w][0])[h * kHeadDim + t], weight, sum);
                }
            }
            sums[h] = sum;
            tops[h] = top;
            dens[h] = den;
        }
        bool finish = true;
        if (units > 1) {
            // leave (sums, maximum, total) of this unit; the last unit of the row's head group to arrive combines them
            float *group_records = scratch + ((size_t)row * q_heads + head0) * kMaxUnits * kRecord;
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                float *mine = group_records + ((size_t)h * kMaxUnits + unit) * kRecord;
                mine[t] = sums[h];
                if (t == 0) {
                    mine[kHeadDim] = tops[h];
                    mine[kHeadDim + 1] = dens[h];
                }
            }
            __threadfence();
            __syncthreads();
            if (t == 0) {
                uint32_t *counter = counters + (size_t)row * groups + kvg;
                const uint32_t before = atomicAdd(counter, 1u);
                arrived = before;
                if (before == (uint32_t)units - 1u) *counter = 0u;  // zero again for the next launch
            }
            __syncthreads();
            finish = arrived == (uint32_t)units - 1u;
            if (finish) {
                __threadfence();
                // weights of the units: one warp per head, lane = unit (at most 8 units)
                for (int h = warp; h < GH; h += kWarps) {
                    const float *all = group_records + (size_t)h * kMaxUnits * kRecord;
                    const float m = lane < units ? __ldcg(all + lane * kRecord + kHeadDim) : -INFINITY;
                    const float l = lane < units ? __ldcg(all + lane * kRecord + kHeadDim + 1) : 0.0f;
                    float top = m;
#pragma unroll
                    for (int d = 16; d > 0; d >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, d));
                    const float weight = lane < units ? exp_approx(__fadd_rn(m, -top)) : 0.0f;
                    float den = __fmul_rn(l, weight);
#pragma unroll
                    for (int d = 16; d > 0; d >>= 1) den = __fadd_rn(den, __shfl_xor_sync(0xffffffffu, den, d));
                    if (lane < kMaxUnits) unit_weight[h][lane] = weight;
                    if (lane == 0) unit_den[h] = den;
                }
                __syncthreads();
                // sums over the units in unit order, all loads in flight at once; thread = channel
#pragma unroll
                for (int h = 0; h < GH; ++h) {
                    const float *all = group_records + (size_t)h * kMaxUnits * kRecord + t;
                    float v[kMaxUnits];
#pragma unroll
                    for (int i = 0; i < kMaxUnits; ++i) v[i] = i < units ? __ldcg(all + i * kRecord) : 0.0f;
                    float sum = 0.0f;
#pragma unroll
                    for (int i = 0; i < kMaxUnits; ++i)
                        if (i < units) sum = __fmaf_rn(v[i], unit_weight[h][i], sum);
                    sums[h] = sum;
                    dens[h] = unit_den[h];
                }
            }
        }
        if (finish) {
            uint32_t row_max = 0;
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                const float v = bf16_rne(__fdiv_rn(sums[h], dens[h]));
                T::store(out + (size_t)row * ldo + (size_t)(head0 + h) * kHeadDim + t, v);
                row_max = max(row_max, absmax_key(v));
            }
            if (maxima) {  // max |out| of the row, for a quantizer that takes its maximum from the producer
                row_max = warp_max_u32(row_max);
                if (lane == 0) atomicMax(maxima + row, row_max);
            }
        }
        __syncthreads();  // the tiles and the per-warp slots are free for the next item; the next ticket has been written
    }
    // every CTA draws exactly one ticket beyond the last item; the CTA that leaves last returns both counters to zero
    if (t == 0) {
        const uint32_t before = atomicAdd(tickets + 1, 1u);
        if (before == gridDim.x - 1u) {
            tickets[0] = 0u;
            tickets[1] = 0u;
        }
    }
}

// ---- greedy selection on stored logits ---------------------------------------------------------------------------
// `select_token` (src/kernels.rs:2191-2231): the largest value, the lowest index among equals, 0xffffffff if any logit
// of the row is not finite.  One CTA of 1024 threads per row; 16-byte loads where the row allows them.
template <class T>
__global__ void __launch_bounds__(1024) select_token_kernel(const typename T::storage *__restrict__ logits, int n, int64_t ld,
                                                            uint32_t *__restrict__ token, float *__restrict__ value, int vector_ok) {
    __shared__ unsigned long long slots[32];
    dependency_wait();
    constexpr int V = T::kVec;
    const int t = threadIdx.x;
    const typename T::storage *x = logits + (size_t)blockIdx.x * ld;
    unsigned long long best = 0;
    if (vector_ok) {
        for (int j = t * V; j < n; j += 1024 * V) {
            float v[V];
            Vec<T>::load(x + j, v);
#pragma unroll
            for (int i = 0; i < V; ++i) best = max(best, argmax_key(v[i], (uint32_t)(j + i)));
        }
    } else {
        for (int j = t; j < n; j += 1024) best = max(best, argmax_key(T::load(x + j), (uint32_t)j));
    }
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
            token[blockIdx.x] = bad ? 0xffffffffu : 0xffffffffu - (uint32_t)(best & 0xffffffffull);
            if (value) {
                const uint32_t o = (uint32_t)(best >> 32);
                const uint32_t bits = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
                value[blockIdx.x] = bad ? __uint_as_float(0x7fc00000u) : __uint_as_float(bits);
            }
        }
    }
}

// Vocabulary split over `parts` ranks: candidates[p] = {rows tokens within part p, rows float32 bit patterns of their
// logits}; the winner per row is the largest value, the lowest part among equals (parts hold ascending token ranges, so
// that is the lowest token id).
__global__ void __launch_bounds__(256) merge_candidates_kernel(const uint32_t *__restrict__ candidates, int parts, int rows, uint32_t part_width,
                                                               uint32_t *__restrict__ token) {
    dependency_wait();
    const int r = blockIdx.x * 256 + threadIdx.x;
    if (r >= rows) return;
    unsigned long long best = 0;
    bool bad = false;
    for (int p = 0; p < parts; ++p) {
        const uint32_t local = candidates[(size_t)(2 * p) * rows + r], bits = candidates[(size_t)(2 * p + 1) * rows + r];
        const unsigned long long key = argmax_key(__uint_as_float(bits), (uint32_t)p);
        if (local == 0xffffffffu || key == ~0ull) bad = true;
        if (key > best) best = key;
    }
    if (bad || best == 0ull) {
        token[r] = 0xffffffffu;
        return;
    }
    const uint32_t p = 0xffffffffu - (uint32_t)(best & 0xffffffffull);
    token[r] = p * part_width + candidates[(size_t)(2 * p) * rows + r];
}

bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Workspace: ticket counters (two words per launch of kMaxRows rows), arrival counters (at most one per (row, head)),
// both padded to 256 bytes and zero between launches, then the partial results of every (row, head, split).
size_t ticket_bytes(int rows) { return ((((size_t)(rows + kMaxRows - 1) / kMaxRows) * 2 * sizeof(uint32_t)) + 255) & ~(size_t)255; }
size_t counter_bytes(int rows, int q_heads) { return (((size_t)rows * q_heads * sizeof(uint32_t)) + 255) & ~(size_t)255; }
size_t workspace_bytes(int rows, int q_heads, int kv_heads) {
    (void)kv_heads;
    return ticket_bytes(rows) + counter_bytes(rows, q_heads) + (size_t)rows * q_heads * kMaxUnits * kRecord * sizeof(float);
}

template <class T, int GH>
cudaError_t launch_batched(const void *q, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache, const uint16_t *v_cache,
                           int64_t cache_stride, const uint32_t *positions, void *out, int64_t ldo, int capacity, uint32_t *maxima,
                           uint32_t *counters, float *scratch, uint32_t *tickets, cudaStream_t s) {
    typedef typename T::storage S;
    // As many CTAs as the GPU holds at once walk the work items (the items are dealt round-robin, so a CTA that had to
    // wait for a free SM would start its share only when others have finished theirs); fewer when the launch cannot have
    // that many items.
    static int per_sm = 0;  // of this instance; the same on every device this library runs on (sm_100a only)
    if (per_sm == 0) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_batched_kernel<T, GH>, kThreads, kSmemBytes);
        if (e != cudaSuccess) return e;
        per_sm = n > 0 ? n : 1;
    }
    const long long most = (long long)rows * kv_heads * ((q_heads / kv_heads) / GH) * ((capacity + kUnitKeys - 1) / kUnitKeys);
    const dim3 grid((unsigned)std::min<long long>(most, (long long)per_sm * sm_count()));
    return launch_kernel(attention_batched_kernel<T, GH>, grid, dim3(kThreads), kSmemBytes, s, (const S *)q, ldq, rows, q_heads, kv_heads, k_cache,
                         v_cache, cache_stride, positions, (S *)out, ldo, capacity, maxima, scratch, counters, tickets, device_status_ptr());
}

template <class T>
cudaError_t launch_batched_any(const void *q, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                               const uint16_t *v_cache, int64_t cache_stride, const uint32_t *positions, void *out, int64_t ldo,
                               int capacity, uint32_t *maxima, uint32_t *counters, float *scratch, uint32_t *tickets, cudaStream_t s) {
    const int group = q_heads / kv_heads;
    if (group % 8 == 0)
        return launch_batched<T, 8>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, cache_stride, positions, out, ldo, capacity, maxima, counters, scratch, tickets, s);
    if (group % 4 == 0)
        return launch_batched<T, 4>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, cache_stride, positions, out, ldo, capacity, maxima, counters, scratch, tickets, s);
    if (group % 2 == 0)
        return launch_batched<T, 2>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, cache_stride, positions, out, ldo, capacity, maxima, counters, scratch, tickets, s);
    return launch_batched<T, 1>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, cache_stride, positions, out, ldo, capacity, maxima, counters, scratch, tickets, s);
}

template <class T> cudaError_t raise_smem() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(attention_batched_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes))) return e;
    if ((e = cudaFuncSetAttribute(attention_batched_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes))) return e;
    if ((e = cudaFuncSetAttribute(attention_batched_kernel<T, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes))) return e;
    return cudaFuncSetAttribute(attention_batched_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
}

}  // namespace

cudaError_t init_batched_decode() {
    cudaError_t e = raise_smem<Bf16>();
    return e == cudaSuccess ? raise_smem<F32>() : e;
}

}  // namespace w8a8

using namespace w8a8;

#define REQUIRE(cond, code)         \
    do {                            \
        if (!(cond)) return (code); \
    } while (0)

extern "C" {

size_t qwen3_attention_batched_workspace(int rows, int q_heads, int kv_heads) {
    if (rows <= 0 || q_heads <= 0 || kv_heads <= 0) return 0;
    return workspace_bytes(rows, q_heads, kv_heads);
}

int qwen3_attention_batched(const void *q, int dtype, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                            const uint16_t *v_cache, int64_t cache_stride, const uint32_t *positions, void *out, int64_t ldo,
                            int capacity, uint32_t *maxima, void *workspace, size_t workspace_size, void *stream) {
    REQUIRE(device_status_ptr(), W8A8_ERR_NOT_INITIALIZED);
    REQUIRE(q && k_cache && v_cache && positions && out && workspace, W8A8_ERR_BAD_ARG);
    REQUIRE(dtype == W8A8_BF16 || dtype == W8A8_F32, W8A8_ERR_BAD_ARG);
    REQUIRE(rows >= 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0, W8A8_ERR_BAD_ARG);
    REQUIRE(capacity > 0 && capacity <= kMaxContext, W8A8_ERR_BAD_ARG);
    REQUIRE(cache_stride >= (int64_t)capacity * kv_heads * kHeadDim, W8A8_ERR_BAD_ARG);
    REQUIRE(ldq >= (int64_t)q_heads * kHeadDim && ldo >= (int64_t)q_heads * kHeadDim, W8A8_ERR_BAD_ARG);
    REQUIRE(aligned(k_cache, 16) && aligned(v_cache, 16) && cache_stride % 8 == 0 && aligned(workspace, 16), W8A8_ERR_ALIGNMENT);
    if (rows == 0) return W8A8_OK;
    REQUIRE(workspace_size >= workspace_bytes(rows, q_heads, kv_heads), W8A8_ERR_BAD_ARG);
    // one launch per kMaxRows rows; the launches run one after the other on the stream and share the workspace
    const size_t esize = dtype == W8A8_BF16 ? 2 : 4;
    uint32_t *tickets = static_cast<uint32_t *>(workspace);
    uint32_t *counters = reinterpret_cast<uint32_t *>(static_cast<char *>(workspace) + ticket_bytes(rows));
    float *scratch = reinterpret_cast<float *>(static_cast<char *>(workspace) + ticket_bytes(rows) + counter_bytes(rows, q_heads));
    for (int r0 = 0; r0 < rows; r0 += kMaxRows) {
        const int n = std::min(kMaxRows, rows - r0);
        const void *qc = static_cast<const char *>(q) + (size_t)r0 * ldq * esize;
        void *oc = static_cast<char *>(out) + (size_t)r0 * ldo * esize;
        const uint16_t *kc = k_cache + (size_t)r0 * cache_stride, *vc = v_cache + (size_t)r0 * cache_stride;
        uint32_t *mc = maxima ? maxima + r0 : nullptr;
        cudaError_t e = dtype == W8A8_BF16
                            ? launch_batched_any<Bf16>(qc, ldq, n, q_heads, kv_heads, kc, vc, cache_stride, positions + r0, oc, ldo, capacity,
                                                       mc, counters + (size_t)r0 * q_heads, scratch + (size_t)r0 * q_heads * kMaxUnits * kRecord,
                                                       tickets + 2 * (r0 / kMaxRows), (cudaStream_t)stream)
                            : launch_batched_any<F32>(qc, ldq, n, q_heads, kv_heads, kc, vc, cache_stride, positions + r0, oc, ldo, capacity,
                                                      mc, counters + (size_t)r0 * q_heads, scratch + (size_t)r0 * q_heads * kMaxUnits * kRecord,
                                                      tickets + 2 * (r0 / kMaxRows), (cudaStream_t)stream);
        if (e != cudaSuccess) return fail_cuda(e, "batched attention launch");
    }
    return W8A8_OK;
}

int qwen3_select_token(const void *logits, int dtype, int rows, int n, int64_t ld, uint32_t *token, float *value, void *stream) {
    REQUIRE(device_status_ptr(), W8A8_ERR_NOT_INITIALIZED);
    REQUIRE(logits && token && rows >= 0 && n > 0 && ld >= n, W8A8_ERR_BAD_ARG);
    REQUIRE(dtype == W8A8_BF16 || dtype == W8A8_F32, W8A8_ERR_BAD_ARG);
    if (rows == 0) return W8A8_OK;
    const int vec = dtype == W8A8_BF16 ? 8 : 4;
    const int vector_ok = aligned(logits, 16) && n % vec == 0 && ld % vec == 0;
    cudaError_t e = dtype == W8A8_BF16
                        ? launch_kernel(select_token_kernel<Bf16>, dim3(rows), dim3(1024), (size_t)0, (cudaStream_t)stream,
                                        (const uint16_t *)logits, n, ld, token, value, vector_ok)
                        : launch_kernel(select_token_kernel<F32>, dim3(rows), dim3(1024), (size_t)0, (cudaStream_t)stream,
                                        (const float *)logits, n, ld, token, value, vector_ok);
    return e == cudaSuccess ? W8A8_OK : fail_cuda(e, "select_token launch");
}

int qwen3_merge_candidates(const uint32_t *candidates, int parts, int rows, int part_width, uint32_t *token, void *stream) {
    REQUIRE(device_status_ptr(), W8A8_ERR_NOT_INITIALIZED);
    REQUIRE(candidates && token && parts > 0 && rows >= 0 && part_width > 0, W8A8_ERR_BAD_ARG);
    if (rows == 0) return W8A8_OK;
    cudaError_t e = launch_kernel(merge_candidates_kernel, dim3((rows + 255) / 256), dim3(256), (size_t)0, (cudaStream_t)stream, candidates,
                                  parts, rows, (uint32_t)part_width, token);
    return e == cudaSuccess ? W8A8_OK : fail_cuda(e, "merge_candidates launch");
}

}  // extern "C"
