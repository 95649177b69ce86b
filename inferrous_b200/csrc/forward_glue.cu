// The operators on either side of the W8A8 linear layers in one Qwen3 decoder layer: token embedding,
// per-head RMSNorm + rotary embedding + KV-cache append, and causal grouped-query attention.
//
// They exist so that the linear-layer kernels can be driven through a whole forward pass (the callers of
// the hot path); they restate the reference's arithmetic (paths under crates/inferrous-qwen3/):
//   embedding    src/kernels.rs:335-345
//   prepare_qk   src/kernels.rs:1350-1443  (= norm :347-413 at width 128, rope :1444-1468, cache :1470-1488)
//   attention    src/kernels.rs:1490-1658  (scores, maximum, exp / total, RN division per key, P.V; the float32
//                sums are reassociated here for parallelism, see the kernel)
// The caches are stored token-major, [position][kv head][128] bf16, for keys and values alike (the reference
// keeps its keys channel-major; the layout is private to these two kernels).
#include "../../include/qwen3_glue.h"
#include "../../include/w8a8.h"
#include "attention_unit.cuh"
#include "common.cuh"
#include "internal.h"

#include <algorithm>

namespace w8a8 {
namespace {

constexpr int kHeadDim = 128;
constexpr int kMaxContext = 4096;  // src/lib.rs:18

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// A value another SM wrote during this kernel: read it from L2.
template <class T> __device__ __forceinline__ float load_cg(const typename T::storage *p);
template <> __device__ __forceinline__ float load_cg<Bf16>(const uint16_t *p) { return bf16_to_f32(__ldcg(p)); }
template <> __device__ __forceinline__ float load_cg<F32>(const float *p) { return __ldcg(p); }

__device__ __forceinline__ void record_range_fault(uint32_t *status, uint32_t detail) {
    if (status && atomicCAS(status, 0u, (uint32_t)FAULT_CACHE_RANGE) == 0u) status[1] = detail;
}

// ---- embedding ---------------------------------------------------------------------------------------------
template <class T>
__global__ void __launch_bounds__(256) embedding_kernel(const uint32_t *__restrict__ ids, const uint16_t *__restrict__ table,
                                                        int hidden, uint32_t vocab, typename T::storage *__restrict__ out,
                                                        uint32_t *status) {
    dependency_wait();
    const int row = blockIdx.y;
    const int c = (blockIdx.x * 256 + threadIdx.x) * 8;
    if (c >= hidden) return;
    const uint32_t id = ids[row];
    if (id >= vocab) {
        if (c == 0) record_range_fault(status, id);
        return;
    }
    float v[8];
    Vec<Bf16>::load(table + (size_t)id * hidden + c, v);
    typename T::storage *o = out + (size_t)row * hidden + c;
    if constexpr (T::kVec == 8) {
        Vec<T>::store(o, v);
    } else {
        const float lo[4] = {v[0], v[1], v[2], v[3]}, hi[4] = {v[4], v[5], v[6], v[7]};
        Vec<T>::store(o, lo);
        Vec<T>::store(o + 4, hi);
    }
}

// ---- head RMSNorm + RoPE + cache append --------------------------------------------------------------------
// One warp per (row, head); lane l holds elements l, l+32, l+64, l+96, so both the reference's first tree
// level ((p[t] + p[t+64]) + (p[t+32] + p[t+96]) for t < 32) and the rotary pairs (t, t+64) are lane-local.
template <class T>
__global__ void __launch_bounds__(128) prepare_qk_kernel(typename T::storage *__restrict__ qkv, int64_t ld, int rows, int q_heads,
                                                         int kv_heads, const float *__restrict__ q_gain,
                                                         const float *__restrict__ k_gain, const float *__restrict__ table,
                                                         const uint32_t *__restrict__ control, uint16_t *__restrict__ k_cache,
                                                         uint16_t *__restrict__ v_cache, int capacity, uint32_t *status,
                                                         const uint32_t *__restrict__ positions, int64_t cache_stride) {
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int per_row = q_heads + kv_heads;
    if (unit >= rows * per_row) return;
    const int row = unit / per_row, h = unit % per_row;
    const bool is_q = h < q_heads;
    // Position, gains and the rotary row do not depend on the preceding kernel (see the note on `control` in the
    // header): they are fetched before the dependency wait.
    // One sequence (positions == nullptr): row r sits at position control[1] + r of the one cache.  Batched decode: row r is
    // the newest token of sequence r, at positions[r] of that sequence's cache (cache_stride elements further on per row).
    const uint32_t pos = positions ? positions[row] : control[1] + (uint32_t)row;
    if (pos >= (uint32_t)capacity) {
        if (lane == 0) record_range_fault(status, pos);
        return;
    }
    if (positions) {
        k_cache += (size_t)row * cache_stride;
        v_cache += (size_t)row * cache_stride;
    }
    const float *gain = is_q ? q_gain : k_gain;
    const float *trow = table + (size_t)pos * kHeadDim;
    float v[4], g[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) g[i] = gain[lane + 32 * i];
    const float c0 = trow[lane], c1 = trow[lane + 32], s0 = trow[lane + 64], s1 = trow[lane + 96];
    dependency_wait();
    typename T::storage *x = qkv + (size_t)row * ld + (size_t)h * kHeadDim;
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = T::load(x + lane + 32 * i);
    float sum = __fadd_rn(__fadd_rn(__fmul_rn(v[0], v[0]), __fmul_rn(v[2], v[2])),
                          __fadd_rn(__fmul_rn(v[1], v[1]), __fmul_rn(v[3], v[3])));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, d));
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float inv = rsqrt_approx(__fadd_rn(__fdiv_rn(sum, 128.0f), 1e-6f));
    float n[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) n[i] = bf16_rne(__fmul_rn(__fmul_rn(v[i], inv), g[i]));
    float r[4];
    r[0] = bf16_rne(__fadd_rn(__fmul_rn(n[0], c0), -__fmul_rn(n[2], s0)));
    r[2] = bf16_rne(__fadd_rn(__fmul_rn(n[2], c0), __fmul_rn(n[0], s0)));
    r[1] = bf16_rne(__fadd_rn(__fmul_rn(n[1], c1), -__fmul_rn(n[3], s1)));
    r[3] = bf16_rne(__fadd_rn(__fmul_rn(n[3], c1), __fmul_rn(n[1], s1)));
    if (is_q) {
#pragma unroll
        for (int i = 0; i < 4; ++i) T::store(x + lane + 32 * i, r[i]);
    } else {
        const int head = h - q_heads;
        const size_t slot = ((size_t)pos * kv_heads + head) * kHeadDim;
        const typename T::storage *vx = qkv + (size_t)row * ld + (size_t)(per_row + head) * kHeadDim;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            T::store(x + lane + 32 * i, r[i]);
            k_cache[slot + lane + 32 * i] = (uint16_t)(__float_as_uint(r[i]) >> 16);
            v_cache[slot + lane + 32 * i] = (uint16_t)(__float_as_uint(T::load(vx + lane + 32 * i)) >> 16);
        }
    }
}

// ---- attention ---------------------------------------------------------------------------------------------
// One CTA of 256 threads per (row, query head, key split).  A split owns a contiguous range of the visible keys;
// with one split the CTA writes the output row itself, otherwise it leaves (maximum, total, unnormalised sums)
// in scratch memory and the last split to arrive combines them (flash-decoding), so that a single decode row
// still spreads over the whole GPU.  The arithmetic of a unit and its association are in attention_unit.cuh.
// The sums are reassociated relative to the reference's one-thread-per-key / one-thread-per-channel kernel (strict
// key and channel order, each weight divided by the total before the P.V sum, src/kernels.rs:1608-1616); the
// association here is fixed by the launch shape and the number of visible keys, so the result depends on nothing
// but the inputs and the launched split count.
constexpr int kAttnThreads = kUnitThreads;
constexpr int kAttnSlices = kUnitSlices;

__device__ __forceinline__ float dot16(const float (&qv)[16], const uint4 a, const uint4 b) { return unit_dot16(qv, a, b); }

template <class T>
__global__ void __launch_bounds__(kAttnThreads) attention_kernel(const typename T::storage *__restrict__ q, int64_t ldq, int q_heads,
                                                                 int kv_heads, const uint16_t *__restrict__ k_cache,
                                                                 const uint16_t *__restrict__ v_cache,
                                                                 const uint32_t *__restrict__ control,
                                                                 typename T::storage *__restrict__ out, int64_t ldo, int capacity,
                                                                 uint32_t *maxima, float *scratch, uint32_t *counters,
                                                                 uint32_t *status, int units, const PrefetchHint hint,
                                                                 int8_t *__restrict__ q_out, float *__restrict__ scale_out) {
    if ((int)blockIdx.x >= units) {
        // Extra CTAs: L2 prefetch hints for weights that a later projection will stream (immutable, so no dependency
        // wait).  The hints are issued and the CTA leaves; the lines arrive while the attention CTAs work.
        if (blockIdx.y == 0) prefetch_ranges(hint, blockIdx.x - units, gridDim.x - units);
        return;
    }
    __shared__ __align__(16) UnitShared sh;
    float *reduce = sh.reduce;
    uint32_t &arrived = sh.arrived;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int unit = blockIdx.x, split = blockIdx.y;
    const int row = unit / q_heads, head = unit % q_heads;
    const int kv = head / (q_heads / kv_heads);
    // The position does not depend on the preceding kernel (see the note on `control` in the header), so the key
    // range of this CTA is known before the dependency wait and its cache lines are pulled towards L2 meanwhile; the
    // one line the preceding kernel is still writing (the newest key) is simply fetched again by the loads below.
    const uint32_t end_u = control[1] + (uint32_t)row + 1u;
    if (end_u > (uint32_t)capacity) {  // every split of the unit takes this branch: nobody waits for anybody
        if (t == 0 && split == 0) record_range_fault(status, end_u);
        return;
    }
    const int end = (int)end_u;
    // Splits in use: one per kAttnKeysPerSplit visible keys, at most the launched number; the rest leave at once.
    int splits, begin, stop;
    unit_range(end, (int)gridDim.y, split, splits, begin, stop);
    if (split >= splits) return;
    const int count = stop - begin;
    {
        const size_t stride_bytes = (size_t)kv_heads * kHeadDim * sizeof(uint16_t);
        const char *kline = reinterpret_cast<const char *>(k_cache) + (size_t)kv * kHeadDim * sizeof(uint16_t);
        const char *vline = reinterpret_cast<const char *>(v_cache) + (size_t)kv * kHeadDim * sizeof(uint16_t);
        for (int i = t; i < 2 * count; i += kAttnThreads) {  // two 128-byte lines per key and per cache
            const size_t off = (size_t)(begin + (i >> 1)) * stride_bytes + (size_t)(i & 1) * 128;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(kline + off));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(vline + off));
        }
    }
    dependency_wait();
    if (t < kHeadDim) sh.query[t] = T::load(q + (size_t)row * ldq + (size_t)head * kHeadDim + t);
    __syncthreads();

    const size_t key_stride = (size_t)kv_heads * kHeadDim;
    const bool wrote = attention_unit<T, false>(sh, SyncCta{}, t, k_cache + (size_t)kv * kHeadDim, v_cache + (size_t)kv * kHeadDim,
                                                key_stride, end, splits, split, begin, stop, (int)gridDim.y, unit, scratch, counters,
                                                out + (size_t)row * ldo + (size_t)head * kHeadDim, maxima ? maxima + row : nullptr);
    if (!wrote) return;
    if (q_out == nullptr) return;

    // Quantizer of the finished row, folded in: the head that completes a row (per-row arrival counter, zero between
    // launches) turns the whole row into int8 codes and its scale, with the arithmetic of `quantize`
    // (src/kernels.rs:415-452): m = max(1e-8, max|x|) ignoring NaN, s = m / 127, q = rne(clamp(x / s)).
    __threadfence();
    __syncthreads();
    if (t == 0) {
        const uint32_t before = atomicAdd(counters + kAttnSplitMaxUnits + row, 1u);
        arrived = before;
        if (before == (uint32_t)q_heads - 1u) counters[kAttnSplitMaxUnits + row] = 0u;
    }
    __syncthreads();
    if (arrived != (uint32_t)q_heads - 1u) return;
    __threadfence();
    const int width = q_heads * kHeadDim;
    const typename T::storage *finished = out + (size_t)row * ldo;
    float m = 1e-8f;
    for (int j = t; j < width; j += kAttnThreads) m = fmaxf(m, fabsf(load_cg<T>(finished + j)));  // fmaxf drops a NaN operand
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    if (lane == 0) reduce[warp] = m;
    __syncthreads();
    m = reduce[0];
#pragma unroll
    for (int i = 1; i < kAttnThreads / 32; ++i) m = fmaxf(m, reduce[i]);
    const float scale = __fdiv_rn(m, 127.0f), inv = __frcp_rn(scale);
    if (t == 0) scale_out[row] = scale;
    int8_t *codes = q_out + (size_t)row * width;
    for (int j = 4 * t; j < width; j += 4 * kAttnThreads) {
        int c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) c[i] = quant_code(load_cg<T>(finished + j + i), scale, inv);
        store_codes<4>(codes + j, c);
    }
}

// ---- attention, many rows (prefill) --------------------------------------------------------------------------
// One CTA of 256 threads per (row, key/value head, group of GH query heads that share it): every key and value is
// read once for the GH heads instead of once per head, which is what bounds the one-head kernel when thousands of
// (row, head) pairs walk the same cache through L2.  Per head the arithmetic and its association are exactly those
// of attention_kernel with one split.  Shared memory: GH * capacity scores (98 KB at 4 heads and 4096 positions).
template <class T, int GH>
__global__ void __launch_bounds__(kAttnThreads) attention_grouped_kernel(const typename T::storage *__restrict__ q, int64_t ldq,
                                                                         int q_heads, int kv_heads,
                                                                         const uint16_t *__restrict__ k_cache,
                                                                         const uint16_t *__restrict__ v_cache,
                                                                         const uint32_t *__restrict__ control,
                                                                         typename T::storage *__restrict__ out, int64_t ldo,
                                                                         int capacity, uint32_t *maxima, uint32_t *status) {
    extern __shared__ __align__(16) float attn_smem[];
    float *scores = attn_smem;                                            // [GH][capacity]
    float(*partial)[GH][kHeadDim] = reinterpret_cast<float(*)[GH][kHeadDim]>(attn_smem + (size_t)GH * capacity);  // [slices]
    float *query = reinterpret_cast<float *>(partial + kAttnSlices);      // [GH][128]
    float *reduce = query + GH * kHeadDim;                                // [warps][GH]
    dependency_wait();
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int group = q_heads / kv_heads;            // query heads per key/value head
    const int chunks = group / GH;                   // CTAs per (row, kv head)
    const int row = blockIdx.x / (kv_heads * chunks);
    const int kv = (blockIdx.x / chunks) % kv_heads;
    const int head0 = kv * group + (blockIdx.x % chunks) * GH;
    const uint32_t end_u = control[1] + (uint32_t)row + 1u;
    if (end_u > (uint32_t)capacity) {
        if (t == 0) record_range_fault(status, end_u);
        return;
    }
    const int end = (int)end_u;
    for (int i = t; i < GH * kHeadDim; i += kAttnThreads)
        query[i] = T::load(q + (size_t)row * ldq + (size_t)head0 * kHeadDim + i);
    __syncthreads();

    const int sub = lane & 7, grp = lane >> 3;
    float qv[GH][16];
#pragma unroll
    for (int h = 0; h < GH; ++h)
#pragma unroll
        for (int i = 0; i < 16; ++i) qv[h][i] = query[h * kHeadDim + 16 * sub + i];
    const size_t key_stride = (size_t)kv_heads * kHeadDim;
    const uint16_t *kbase = k_cache + (size_t)kv * kHeadDim + 16 * sub;
    float maximum[GH];
#pragma unroll
    for (int h = 0; h < GH; ++h) maximum[h] = -INFINITY;
#pragma unroll 2
    for (int j0 = warp * 4; j0 < end; j0 += (kAttnThreads / 32) * 4) {
        const int j = j0 + grp;
        uint4 a = make_uint4(0, 0, 0, 0), b = a;
        if (j < end) {
            const uint4 *kr = reinterpret_cast<const uint4 *>(kbase + (size_t)j * key_stride);
            a = kr[0];
            b = kr[1];
        }
#pragma unroll
        for (int h = 0; h < GH; ++h) {
            float s = j < end ? dot16(qv[h], a, b) : 0.0f;
            s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 4));
            s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
            s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
            s = __fmul_rn(s, 0.08838834764831845f);
            if (j < end) {
                maximum[h] = fmaxf(maximum[h], s);
                if (sub == 0) scores[(size_t)h * capacity + j] = s;
            }
        }
    }
#pragma unroll
    for (int h = 0; h < GH; ++h) {
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) maximum[h] = fmaxf(maximum[h], __shfl_xor_sync(0xffffffffu, maximum[h], d));
        if (lane == 0) reduce[warp * GH + h] = maximum[h];
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < GH; ++h) {
        maximum[h] = reduce[h];
#pragma unroll
        for (int i = 1; i < kAttnThreads / 32; ++i) maximum[h] = fmaxf(maximum[h], reduce[i * GH + h]);
    }
    __syncthreads();

    float total[GH];
#pragma unroll
    for (int h = 0; h < GH; ++h) {
        total[h] = 0.0f;
        float *sc = scores + (size_t)h * capacity;
        for (int j = t; j < end; j += kAttnThreads) {
            const float e = exp_approx(__fadd_rn(sc[j], -maximum[h]));
            sc[j] = e;
            total[h] = __fadd_rn(total[h], e);
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) total[h] = __fadd_rn(total[h], __shfl_xor_sync(0xffffffffu, total[h], d));
        if (lane == 0) reduce[warp * GH + h] = total[h];
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < GH; ++h) {
        total[h] = reduce[h];
#pragma unroll
        for (int i = 1; i < kAttnThreads / 32; ++i) total[h] = __fadd_rn(total[h], reduce[i * GH + h]);
    }

    const int slice = t >> 4, cg = t & 15;
    const uint16_t *vbase = v_cache + (size_t)kv * kHeadDim + 8 * cg;
    float acc[GH][8];
#pragma unroll
    for (int h = 0; h < GH; ++h)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[h][i] = 0.0f;
#pragma unroll 2
    for (int j = slice; j < end; j += kAttnSlices) {
        const uint4 v = *reinterpret_cast<const uint4 *>(vbase + (size_t)j * key_stride);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int h = 0; h < GH; ++h) {
            const float p = scores[(size_t)h * capacity + j];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[h][2 * i] = __fadd_rn(acc[h][2 * i], __fmul_rn(p, __uint_as_float(w[i] << 16)));
                acc[h][2 * i + 1] = __fadd_rn(acc[h][2 * i + 1], __fmul_rn(p, __uint_as_float(w[i] & 0xffff0000u)));
            }
        }
    }
#pragma unroll
    for (int h = 0; h < GH; ++h)
#pragma unroll
        for (int i = 0; i < 8; ++i) partial[slice][h][8 * cg + i] = acc[h][i];
    __syncthreads();
    // GH * 128 outputs over 256 threads
    for (int o = t; o < GH * kHeadDim; o += kAttnThreads) {
        const int h = o / kHeadDim, c = o % kHeadDim;
        float sum = partial[0][h][c];
#pragma unroll
        for (int i = 1; i < kAttnSlices; ++i) sum = __fadd_rn(sum, partial[i][h][c]);
        float den = total[0];
#pragma unroll
        for (int k = 1; k < GH; ++k)
            if (h == k) den = total[k];
        const float v = bf16_rne(__fdiv_rn(sum, den));
        T::store(out + (size_t)row * ldo + (size_t)(head0 + h) * kHeadDim + c, v);
        if (maxima) {
            const uint32_t m = warp_max_u32(absmax_key(v));
            if (lane == 0) atomicMax(maxima + row, m);
        }
    }
}

// ---- attention, many rows, on the tensor cores -----------------------------------------------------------------
// Prefill of 32 rows or more: one CTA of 4 warps per (block of 64 rows, query head), each warp 16 rows, keys and values
// staged 64 at a time in shared memory, both products on mma.sync.m16n8k16 (bf16 x bf16 -> f32), running maximum and
// total per row (flash attention).  What keeps it inside the same bound as the CUDA-core kernels:
//   * q, k and v ARE bf16 values, so Q.K^T has exact products and float32 sums (association differs, nothing else);
//   * the softmax weights are float32; each enters the P.V product as hi + lo, two bf16 numbers with hi = bf16(p) and
//     lo = bf16(p - hi), so p is carried to 16 mantissa bits instead of 8 and the second product costs one more MMA;
//   * exp is the same ex2.approx form, the division by the total happens once at the end.
// This is the one place where the library uses the legacy warp-level MMA: a 16 x 64 score tile per warp is far below
// the 128-row granularity of tcgen05, and attention is not on the W8A8 path.
constexpr int kMmaRows = 64;     // rows per CTA
constexpr int kMmaKeys = 64;     // keys per shared-memory tile
constexpr int kMmaPitch = kHeadDim + 8;  // bf16 elements per staged row: 272 bytes, conflict-free for the fragment loads
constexpr size_t kMmaSmemBytes = (size_t)2 * 2 * kMmaKeys * kMmaPitch * sizeof(uint16_t);  // 2 stages x {K, V}: 68 KiB

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {  // both already bf16-representable
    return (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xffff0000u);
}
template <class T> __device__ __forceinline__ uint32_t load_pair(const typename T::storage *p);
template <> __device__ __forceinline__ uint32_t load_pair<Bf16>(const uint16_t *p) { return *reinterpret_cast<const uint32_t *>(p); }
template <> __device__ __forceinline__ uint32_t load_pair<F32>(const float *p) {
    const float2 v = *reinterpret_cast<const float2 *>(p);
    return pack_bf16(v.x, v.y);
}
template <class T> __device__ __forceinline__ void store_pair(typename T::storage *p, float a, float b);
template <> __device__ __forceinline__ void store_pair<Bf16>(uint16_t *p, float a, float b) { *reinterpret_cast<uint32_t *>(p) = pack_bf16(a, b); }
template <> __device__ __forceinline__ void store_pair<F32>(float *p, float a, float b) { *reinterpret_cast<float2 *>(p) = make_float2(a, b); }

template <class T>
__global__ void __launch_bounds__(128) attention_mma_kernel(const typename T::storage *__restrict__ q, int64_t ldq, int rows, int q_heads,
                                                            int kv_heads, const uint16_t *__restrict__ k_cache,
                                                            const uint16_t *__restrict__ v_cache,
                                                            const uint32_t *__restrict__ control,
                                                            typename T::storage *__restrict__ out, int64_t ldo, int capacity,
                                                            uint32_t *maxima, uint32_t *status) {
    // two stages of {keys, values}: the next tile is copied (cp.async) while the current one is multiplied
    extern __shared__ __align__(16) uint16_t mma_smem[];
    typedef uint16_t (*TilePtr)[kMmaPitch];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31, g = lane >> 2, tq = lane & 3;
    const int head = blockIdx.y, kv = head / (q_heads / kv_heads);
    // causal attention: the last row blocks see the most keys, so they are scheduled first
    const int row0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kMmaRows;  // first row of the CTA
    const int last_row = min(rows, row0 + kMmaRows) - 1;       // last valid row of the CTA
    const uint32_t position = control[1];
    if (position + (uint32_t)rows > (uint32_t)capacity) {      // the same verdict in every CTA of the launch
        if (t == 0 && row0 == 0 && head == 0) record_range_fault(status, position + (uint32_t)rows);
        return;
    }
    dependency_wait();
    const int r_lo = row0 + warp * 16 + g, r_hi = r_lo + 8;   // the two rows this thread holds
    const int rl = min(r_lo, rows - 1), rh = min(r_hi, rows - 1);  // clamped for loads; stores are guarded
    // Q fragments: 8 steps of 16 channels
    uint32_t qa[8][4];
    {
        const typename T::storage *ql = q + (size_t)rl * ldq + (size_t)head * kHeadDim + 2 * tq;
        const typename T::storage *qh = q + (size_t)rh * ldq + (size_t)head * kHeadDim + 2 * tq;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            qa[s][0] = load_pair<T>(ql + 16 * s);
            qa[s][1] = load_pair<T>(qh + 16 * s);
            qa[s][2] = load_pair<T>(ql + 16 * s + 8);
            qa[s][3] = load_pair<T>(qh + 16 * s + 8);
        }
    }
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.0f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
    const int end_cta = (int)position + last_row + 1;          // keys visible to the CTA's last row
    const int vis_lo = (int)position + r_lo, vis_hi = (int)position + r_hi;  // last visible key of each row
    const size_t key_stride = (size_t)kv_heads * kHeadDim;

    auto stage = [&](int buf, int k0) {  // 16 vectors of 16 bytes per key and per cache; keys past the end are zeros
        TilePtr kd = reinterpret_cast<TilePtr>(mma_smem + (size_t)buf * 2 * kMmaKeys * kMmaPitch);
        TilePtr vd = kd + kMmaKeys;
        for (int i = t; i < kMmaKeys * (kHeadDim / 8); i += 128) {
            const int key = i >> 4, part = i & 15;
            if (k0 + key < end_cta) {
                const size_t off = (size_t)(k0 + key) * key_stride + (size_t)kv * kHeadDim + 8 * part;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&kd[key][8 * part])), "l"(k_cache + off));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&vd[key][8 * part])), "l"(v_cache + off));
            } else {
                *reinterpret_cast<uint4 *>(&kd[key][8 * part]) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(&vd[key][8 * part]) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    int buf = 0;
    for (int k0 = 0; k0 < end_cta; k0 += kMmaKeys, buf ^= 1) {
        const bool more = k0 + kMmaKeys < end_cta;
        if (more) stage(buf ^ 1, k0 + kMmaKeys);  // that buffer was released by the barrier that ended the previous iteration
        if (more)
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        else
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // tile k0 has landed for every thread
        TilePtr ks = reinterpret_cast<TilePtr>(mma_smem + (size_t)buf * 2 * kMmaKeys * kMmaPitch);
        TilePtr vs = ks + kMmaKeys;
        if (k0 <= (int)position + row0 + warp * 16 + 15) {  // else: no key of this tile is visible to this warp's rows
            // scores of 16 rows x 64 keys
            float sc[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int i = 0; i < 4; ++i) sc[n][i] = 0.0f;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(&ks[n * 8 + g][16 * s + 2 * tq]);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t *>(&ks[n * 8 + g][16 * s + 2 * tq + 8]);
                    mma_bf16(sc[n], qa[s], b0, b1);
                }
            }
            // scale, causal mask, running maximum
            float t_lo = -INFINITY, t_hi = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const int key = k0 + n * 8 + 2 * tq;
                sc[n][0] = key <= vis_lo ? __fmul_rn(sc[n][0], 0.08838834764831845f) : -INFINITY;
                sc[n][1] = key + 1 <= vis_lo ? __fmul_rn(sc[n][1], 0.08838834764831845f) : -INFINITY;
                sc[n][2] = key <= vis_hi ? __fmul_rn(sc[n][2], 0.08838834764831845f) : -INFINITY;
                sc[n][3] = key + 1 <= vis_hi ? __fmul_rn(sc[n][3], 0.08838834764831845f) : -INFINITY;
                t_lo = fmaxf(t_lo, fmaxf(sc[n][0], sc[n][1]));
                t_hi = fmaxf(t_hi, fmaxf(sc[n][2], sc[n][3]));
            }
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1));
            t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1));
            t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
            const float n_lo = fmaxf(m_lo, t_lo), n_hi = fmaxf(m_hi, t_hi);
            // a row with nothing visible yet keeps maximum -inf: its weights are 0 and nothing is rescaled
            const float c_lo = n_lo == -INFINITY ? 1.0f : exp_approx(__fadd_rn(m_lo, -n_lo));
            const float c_hi = n_hi == -INFINITY ? 1.0f : exp_approx(__fadd_rn(m_hi, -n_hi));
            const float b_lo = n_lo == -INFINITY ? 0.0f : n_lo, b_hi = n_hi == -INFINITY ? 0.0f : n_hi;
            m_lo = n_lo;
            m_hi = n_hi;
            l_lo = __fmul_rn(l_lo, c_lo);
            l_hi = __fmul_rn(l_hi, c_hi);
#pragma unroll
            for (int n = 0; n < 16; ++n) {
                o[n][0] = __fmul_rn(o[n][0], c_lo);
                o[n][1] = __fmul_rn(o[n][1], c_lo);
                o[n][2] = __fmul_rn(o[n][2], c_hi);
                o[n][3] = __fmul_rn(o[n][3], c_hi);
            }
            // weights, split into two bf16 parts, and the P.V product
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // 16 keys per step: score tiles 2j and 2j+1
                uint32_t ph[4], pl[4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float p[4];
                    p[0] = exp_approx(__fadd_rn(sc[2 * j + h][0], -b_lo));
                    p[1] = exp_approx(__fadd_rn(sc[2 * j + h][1], -b_lo));
                    p[2] = exp_approx(__fadd_rn(sc[2 * j + h][2], -b_hi));
                    p[3] = exp_approx(__fadd_rn(sc[2 * j + h][3], -b_hi));
                    l_lo = __fadd_rn(l_lo, __fadd_rn(p[0], p[1]));
                    l_hi = __fadd_rn(l_hi, __fadd_rn(p[2], p[3]));
                    float hi[4], lo[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        hi[i] = bf16_rne(p[i]);
                        lo[i] = bf16_rne(__fadd_rn(p[i], -hi[i]));
                    }
                    ph[2 * h] = pack_bf16(hi[0], hi[1]);
                    ph[2 * h + 1] = pack_bf16(hi[2], hi[3]);
                    pl[2 * h] = pack_bf16(lo[0], lo[1]);
                    pl[2 * h + 1] = pack_bf16(lo[2], lo[3]);
                }
                const uint32_t vrow = smem_addr(&vs[16 * j + (lane & 15)][0]);
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    uint32_t b0, b1;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(vrow + 16u * n));
                    mma_bf16(o[n], ph, b0, b1);
                    mma_bf16(o[n], pl, b0, b1);
                }
            }
        }
        __syncthreads();  // every warp is done with this buffer; the next iteration refills it
    }
    // totals over the four lanes that share a row, then the one division
    l_lo = __fadd_rn(l_lo, __shfl_xor_sync(0xffffffffu, l_lo, 1));
    l_lo = __fadd_rn(l_lo, __shfl_xor_sync(0xffffffffu, l_lo, 2));
    l_hi = __fadd_rn(l_hi, __shfl_xor_sync(0xffffffffu, l_hi, 1));
    l_hi = __fadd_rn(l_hi, __shfl_xor_sync(0xffffffffu, l_hi, 2));
    uint32_t mx_lo = 0, mx_hi = 0;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
        const float a0 = bf16_rne(__fdiv_rn(o[n][0], l_lo)), a1 = bf16_rne(__fdiv_rn(o[n][1], l_lo));
        const float a2 = bf16_rne(__fdiv_rn(o[n][2], l_hi)), a3 = bf16_rne(__fdiv_rn(o[n][3], l_hi));
        if (r_lo < rows) store_pair<T>(out + (size_t)r_lo * ldo + (size_t)head * kHeadDim + 8 * n + 2 * tq, a0, a1);
        if (r_hi < rows) store_pair<T>(out + (size_t)r_hi * ldo + (size_t)head * kHeadDim + 8 * n + 2 * tq, a2, a3);
        mx_lo = max(mx_lo, max(absmax_key(a0), absmax_key(a1)));
        mx_hi = max(mx_hi, max(absmax_key(a2), absmax_key(a3)));
    }
    if (maxima) {
        mx_lo = max(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = max(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = max(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = max(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        if (tq == 0 && r_lo < rows) atomicMax(maxima + r_lo, mx_lo);
        if (tq == 0 && r_hi < rows) atomicMax(maxima + r_hi, mx_hi);
    }
}

size_t grouped_smem(int gh, int capacity) {
    return ((size_t)gh * capacity + (size_t)kAttnSlices * gh * kHeadDim + (size_t)gh * kHeadDim + (kAttnThreads / 32) * gh) * sizeof(float);
}

template <class T, int GH>
cudaError_t launch_grouped(const typename T::storage *q, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                           const uint16_t *v_cache, const uint32_t *control, typename T::storage *out, int64_t ldo, int capacity,
                           uint32_t *maxima, cudaStream_t s) {
    const size_t smem = grouped_smem(GH, capacity);
    const dim3 grid(rows * kv_heads * ((q_heads / kv_heads) / GH));
    return launch_kernel(attention_grouped_kernel<T, GH>, grid, dim3(kAttnThreads), smem, s, q, ldq, q_heads, kv_heads, k_cache,
                         v_cache, control, out, ldo, capacity, maxima, device_status_ptr());
}

template <class T>
cudaError_t launch_grouped_any(const void *q, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                               const uint16_t *v_cache, const uint32_t *control, void *out, int64_t ldo, int capacity,
                               uint32_t *maxima, cudaStream_t s) {
    typedef typename T::storage S;
    const int group = q_heads / kv_heads;
    if (group % 4 == 0)
        return launch_grouped<T, 4>((const S *)q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, control, (S *)out, ldo, capacity, maxima, s);
    if (group % 2 == 0)
        return launch_grouped<T, 2>((const S *)q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, control, (S *)out, ldo, capacity, maxima, s);
    return launch_grouped<T, 1>((const S *)q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, control, (S *)out, ldo, capacity, maxima, s);
}

bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

constexpr int kMmaMinRows = 32;
bool g_attention_no_mma = false;  // test switch (qwen3_attention_use_tensor_cores): keep many-row launches on the CUDA cores

template <class T> cudaError_t raise_grouped_smem() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(attention_grouped_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)grouped_smem(1, kMaxContext)))) return e;
    if ((e = cudaFuncSetAttribute(attention_grouped_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)grouped_smem(2, kMaxContext)))) return e;
    return cudaFuncSetAttribute(attention_grouped_kernel<T, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)grouped_smem(4, kMaxContext));
}

}  // namespace

cudaError_t init_forward_glue() {
    cudaError_t e = raise_grouped_smem<Bf16>();
    if (e == cudaSuccess) e = raise_grouped_smem<F32>();
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_mma_kernel<Bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_mma_kernel<F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmemBytes);
    return e;
}

}  // namespace w8a8

using namespace w8a8;

#define REQUIRE(cond, code)         \
    do {                            \
        if (!(cond)) return (code); \
    } while (0)

extern "C" {

int qwen3_embedding(const uint32_t *ids, const uint16_t *table, int rows, int hidden, int vocab, void *out, int dtype, void *stream) {
    REQUIRE(device_status_ptr(), W8A8_ERR_NOT_INITIALIZED);
    REQUIRE(ids && table && out && rows >= 0 && hidden > 0 && vocab > 0, W8A8_ERR_BAD_ARG);
    REQUIRE(dtype == W8A8_BF16 || dtype == W8A8_F32, W8A8_ERR_BAD_ARG);
    REQUIRE(hidden % 8 == 0 && aligned(table, 16) && aligned(out, 16), W8A8_ERR_ALIGNMENT);
    if (rows == 0) return W8A8_OK;
    const dim3 grid((hidden / 8 + 255) / 256, rows);
    cudaError_t e = dtype == W8A8_BF16
                        ? launch_kernel(embedding_kernel<Bf16>, grid, dim3(256), 0, (cudaStream_t)stream, ids, table, hidden,
                                        (uint32_t)vocab, (uint16_t *)out, device_status_ptr())
                        : launch_kernel(embedding_kernel<F32>, grid, dim3(256), 0, (cudaStream_t)stream, ids, table, hidden,
                                        (uint32_t)vocab, (float *)out, device_status_ptr());
    return e == cudaSuccess ? W8A8_OK : fail_cuda(e, "embedding launch");
}

static int prepare_qk_impl(void *qkv, int dtype, int64_t ld, int rows, int q_heads, int kv_heads, const float *q_gain,
                           const float *k_gain, const float *rope_table, const uint32_t *control, const uint32_t *positions,
                           int64_t cache_stride, uint16_t *k_cache, uint16_t *v_cache, int capacity, void *stream) {
    REQUIRE(device_status_ptr(), W8A8_ERR_NOT_INITIALIZED);
    REQUIRE(qkv && q_gain && k_gain && rope_table && (control || positions) && k_cache && v_cache, W8A8_ERR_BAD_ARG);
    REQUIRE(dtype == W8A8_BF16 || dtype == W8A8_F32, W8A8_ERR_BAD_ARG);
    REQUIRE(rows >= 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0, W8A8_ERR_BAD_ARG);
    REQUIRE(capacity > 0 && capacity <= kMaxContext && ld >= (int64_t)(q_heads + 2 * kv_heads) * kHeadDim, W8A8_ERR_BAD_ARG);
    if (rows == 0) return W8A8_OK;
    const int units = rows * (q_heads + kv_heads);
    const dim3 grid((units + 3) / 4);
    cudaError_t e =
        dtype == W8A8_BF16
            ? launch_kernel(prepare_qk_kernel<Bf16>, grid, dim3(128), 0, (cudaStream_t)stream, (uint16_t *)qkv, ld, rows, q_heads,
                            kv_heads, q_gain, k_gain, rope_table, control, k_cache, v_cache, capacity, device_status_ptr(), positions,
                            cache_stride)
            : launch_kernel(prepare_qk_kernel<F32>, grid, dim3(128), 0, (cudaStream_t)stream, (float *)qkv, ld, rows, q_heads,
                            kv_heads, q_gain, k_gain, rope_table, control, k_cache, v_cache, capacity, device_status_ptr(), positions,
                            cache_stride);
    return e == cudaSuccess ? W8A8_OK : fail_cuda(e, "prepare_qk launch");
}

int qwen3_prepare_qk(void *qkv, int dtype, int64_t ld, int rows, int q_heads, int kv_heads, const float *q_gain,
                     const float *k_gain, const float *rope_table, const uint32_t *control, uint16_t *k_cache, uint16_t *v_cache,
                     int capacity, void *stream) {
    REQUIRE(control, W8A8_ERR_BAD_ARG);
    return prepare_qk_impl(qkv, dtype, ld, rows, q_heads, kv_heads, q_gain, k_gain, rope_table, control, nullptr, 0, k_cache, v_cache,
                           capacity, stream);
}

int qwen3_prepare_qk_batched(void *qkv, int dtype, int64_t ld, int rows, int q_heads, int kv_heads, const float *q_gain,
                             const float *k_gain, const float *rope_table, const uint32_t *positions, uint16_t *k_cache,
                             uint16_t *v_cache, int capacity, int64_t cache_stride, void *stream) {
    REQUIRE(positions && cache_stride >= (int64_t)capacity * kv_heads * kHeadDim, W8A8_ERR_BAD_ARG);
    return prepare_qk_impl(qkv, dtype, ld, rows, q_heads, kv_heads, q_gain, k_gain, rope_table, nullptr, positions, cache_stride, k_cache,
                           v_cache, capacity, stream);
}

static int attention_impl(const void *q, int dtype, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                          const uint16_t *v_cache, const uint32_t *control, void *out, int64_t ldo, int capacity, uint32_t *maxima,
                          int8_t *q_out, float *scale_out, void *stream) {
    REQUIRE(device_status_ptr(), W8A8_ERR_NOT_INITIALIZED);
    REQUIRE(q && k_cache && v_cache && control && out, W8A8_ERR_BAD_ARG);
    REQUIRE(dtype == W8A8_BF16 || dtype == W8A8_F32, W8A8_ERR_BAD_ARG);
    REQUIRE(rows >= 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0, W8A8_ERR_BAD_ARG);
    REQUIRE(capacity > 0 && capacity <= kMaxContext, W8A8_ERR_BAD_ARG);
    REQUIRE(ldq >= (int64_t)q_heads * kHeadDim && ldo >= (int64_t)q_heads * kHeadDim, W8A8_ERR_BAD_ARG);
    REQUIRE(aligned(k_cache, 16) && aligned(v_cache, 16), W8A8_ERR_ALIGNMENT);
    if (rows == 0) return W8A8_OK;
    // Few (row, head) units: split the keys of each over several CTAs, at most two CTAs per SM in all.
    const int units = rows * q_heads;
    int splits = 1;
    if (units < sm_count() && units <= kAttnSplitMaxUnits) splits = attention_splits(units);
    // the folded quantizer exists in the few-row kernel only
    REQUIRE(q_out == nullptr || (rows * q_heads < sm_count() && rows * q_heads <= kAttnSplitMaxUnits), W8A8_ERR_UNSUPPORTED);
    if (rows >= kMmaMinRows && (ldq % 2) == 0 && (ldo % 2) == 0 && aligned(q, 8) && aligned(out, 8) && !g_attention_no_mma) {
        // prefill: tensor-core kernel, 64 rows per CTA
        const dim3 grid_mma((rows + kMmaRows - 1) / kMmaRows, q_heads);
        cudaError_t em = dtype == W8A8_BF16
                             ? launch_kernel(attention_mma_kernel<Bf16>, grid_mma, dim3(128), kMmaSmemBytes, (cudaStream_t)stream, (const uint16_t *)q,
                                             ldq, rows, q_heads, kv_heads, k_cache, v_cache, control, (uint16_t *)out, ldo, capacity,
                                             maxima, device_status_ptr())
                             : launch_kernel(attention_mma_kernel<F32>, grid_mma, dim3(128), kMmaSmemBytes, (cudaStream_t)stream, (const float *)q,
                                             ldq, rows, q_heads, kv_heads, k_cache, v_cache, control, (float *)out, ldo, capacity,
                                             maxima, device_status_ptr());
        return em == cudaSuccess ? W8A8_OK : fail_cuda(em, "attention launch");
    }
    if (splits == 1 && units >= sm_count()) {
        // many rows: one CTA per (row, key/value head) serves the query heads that share it
        cudaError_t eg = dtype == W8A8_BF16
                             ? launch_grouped_any<Bf16>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, control, out, ldo, capacity,
                                                        maxima, (cudaStream_t)stream)
                             : launch_grouped_any<F32>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, control, out, ldo, capacity,
                                                       maxima, (cudaStream_t)stream);
        return eg == cudaSuccess ? W8A8_OK : fail_cuda(eg, "attention launch");
    }
    const PrefetchHint hint = take_prefetch_hint();
    const int prefetch_ctas = hint.count ? sm_count() : 0;
    const dim3 grid(units + prefetch_ctas, splits);
    cudaError_t e = dtype == W8A8_BF16
                        ? launch_kernel(attention_kernel<Bf16>, grid, dim3(kAttnThreads), 0, (cudaStream_t)stream, (const uint16_t *)q, ldq,
                                        q_heads, kv_heads, k_cache, v_cache, control, (uint16_t *)out, ldo, capacity, maxima,
                                        attention_scratch(), attention_counters(), device_status_ptr(), units, hint, q_out, scale_out)
                        : launch_kernel(attention_kernel<F32>, grid, dim3(kAttnThreads), 0, (cudaStream_t)stream, (const float *)q, ldq,
                                        q_heads, kv_heads, k_cache, v_cache, control, (float *)out, ldo, capacity, maxima,
                                        attention_scratch(), attention_counters(), device_status_ptr(), units, hint, q_out, scale_out);
    return e == cudaSuccess ? W8A8_OK : fail_cuda(e, "attention launch");
}

int qwen3_attention(const void *q, int dtype, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                    const uint16_t *v_cache, const uint32_t *control, void *out, int64_t ldo, int capacity, uint32_t *maxima,
                    void *stream) {
    return attention_impl(q, dtype, ldq, rows, q_heads, kv_heads, k_cache, v_cache, control, out, ldo, capacity, maxima, nullptr,
                          nullptr, stream);
}

int qwen3_attention_quantize(const void *q, int dtype, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                             const uint16_t *v_cache, const uint32_t *control, void *out, int64_t ldo, int capacity,
                             int8_t *codes, float *scale, void *stream) {
    REQUIRE(codes && scale && (reinterpret_cast<uintptr_t>(codes) & 3u) == 0, W8A8_ERR_BAD_ARG);
    return attention_impl(q, dtype, ldq, rows, q_heads, kv_heads, k_cache, v_cache, control, out, ldo, capacity, nullptr, codes,
                          scale, stream);
}

int qwen3_attention_use_tensor_cores(int enabled) {
    g_attention_no_mma = enabled == 0;
    return W8A8_OK;
}

}  // extern "C"
