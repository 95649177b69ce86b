// One (query head, key split) unit of split-key decode attention, as a device function of 256 threads.
//
// Two kernels run it: attention_kernel (forward_glue.cu; one CTA per unit) and the resident decode kernel
// (decode_layers.cu; two units side by side in a CTA of 512 threads).  Both must give the same bits for the same
// inputs and launched split count, which is why the arithmetic lives here once:
//   scores   eight lanes per key (16 channels each, summed in order, then a three-step butterfly), four keys per
//            warp and sweep; score = dot * 128^-0.5, as the reference scales it (src/kernels.rs:1490-1658)
//   softmax  e = exp(score - maximum) with the reference's ex2.approx form; total = sum of e
//   P.V      sixteen key slices (key j belongs to slice j % 16) x sixteen lanes of 8 channels, each slice summed
//            in increasing j, the sixteen partial sums added in slice order; one RN division by the total at the end
//   combine  maximum M over the splits, weights exp(m_s - M), sums and totals added in split order, one division
// The association is fixed by the 256 threads, the number of visible keys and the launched split count.
#pragma once
#include "common.cuh"

namespace w8a8 {

constexpr int kUnitThreads = 256;
constexpr int kUnitSlices = 16;
constexpr int kUnitHeadDim = 128;
constexpr int kUnitRecord = kUnitHeadDim + 4;  // floats per (unit, split) in scratch: 128 sums, maximum, total, padding
constexpr int kUnitKeysPerSplit = 64;          // a split is not worth its combine step for fewer keys
constexpr int kUnitMaxContext = 4096;          // src/lib.rs:18

// Shared memory of one unit (the caller provides it; 16-byte aligned).
struct UnitShared {
    float scores[kUnitMaxContext];
    float partial[kUnitSlices][kUnitHeadDim];
    float query[kUnitHeadDim];                 // the head's query row (after head norm and rotary embedding)
    float reduce[kUnitThreads / 32];
    uint32_t arrived;
    uint32_t pad[3];
    uint16_t fresh_k[kUnitHeadDim];            // FRESH: the newest key / value of the head, not yet in the cache
    uint16_t fresh_v[kUnitHeadDim];
};

struct SyncCta {  // all threads of the CTA belong to the unit
    __device__ __forceinline__ void operator()() const { __syncthreads(); }
};
struct SyncNamed {  // 256 threads of a larger CTA, on a named barrier
    int id;
    __device__ __forceinline__ void operator()() const { asm volatile("bar.sync %0, 256;" ::"r"(id) : "memory"); }
};

__device__ __forceinline__ float unit_dot16(const float (&qv)[16], const uint4 a, const uint4 b) {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        s = __fadd_rn(s, __fmul_rn(qv[2 * i], __uint_as_float(w[i] << 16)));
        s = __fadd_rn(s, __fmul_rn(qv[2 * i + 1], __uint_as_float(w[i] & 0xffff0000u)));
    }
    return s;
}

// Splits in use and this split's key range for `end` visible keys and `launched` splits.
__device__ __forceinline__ void unit_range(int end, int launched, int split, int &splits, int &begin, int &stop) {
    splits = min(launched, (end + kUnitKeysPerSplit - 1) / kUnitKeysPerSplit);
    const int chunk = (((end + splits - 1) / splits) + 31) & ~31;  // ranges of a multiple of 32 keys
    begin = min(end, split * chunk);
    stop = min(end, begin + chunk);
}

// t = thread within the unit (0..255).  sh.query holds the query row.  The caches are [position][kv head][128] bf16 and
// `k_head` / `v_head` point at position 0 of this unit's key/value head.  FRESH: key and value `end - 1` are taken
// from sh.fresh_k / sh.fresh_v instead of the cache.  Returns true in the threads of the unit that wrote the head's
// output (one split, or the last split to arrive); `out_head` receives 128 values, `maxima_row` (optional) max |out|.
template <class T, bool FRESH, class Sync>
__device__ __forceinline__ bool attention_unit(UnitShared &sh, const Sync sync, int t, const uint16_t *__restrict__ k_head,
                                               const uint16_t *__restrict__ v_head, size_t key_stride, int end, int splits,
                                               int split, int begin, int stop, int launched, int unit, float *scratch,
                                               uint32_t *counters, typename T::storage *__restrict__ out_head,
                                               uint32_t *maxima_row) {
    const int warp = t >> 5, lane = t & 31;
    const int count = stop - begin;
    const int newest = end - 1 - begin;  // FRESH: index within this split of the key that is not in the cache yet

    // scores
    const int sub = lane & 7, group = lane >> 3;
    float qv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) qv[i] = sh.query[16 * sub + i];
    const uint16_t *kbase = k_head + (size_t)begin * key_stride + 16 * sub;
    float maximum = -INFINITY;
#pragma unroll 2
    for (int j0 = warp * 4; j0 < count; j0 += (kUnitThreads / 32) * 4) {
        const int j = j0 + group;
        float s = 0.0f;
        if (j < count) {
            const uint4 *kr = reinterpret_cast<const uint4 *>(kbase + (size_t)j * key_stride);
            if (FRESH && j == newest) kr = reinterpret_cast<const uint4 *>(sh.fresh_k + 16 * sub);
            s = unit_dot16(qv, kr[0], kr[1]);
        }
        s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 4));
        s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
        s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
        s = __fmul_rn(s, 0.08838834764831845f);
        if (j < count) {
            maximum = fmaxf(maximum, s);
            if (sub == 0) sh.scores[j] = s;
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, d));
    if (lane == 0) sh.reduce[warp] = maximum;
    sync();
    maximum = sh.reduce[0];
#pragma unroll
    for (int i = 1; i < kUnitThreads / 32; ++i) maximum = fmaxf(maximum, sh.reduce[i]);
    sync();

    // softmax numerators and their total (an empty split has maximum -inf and total 0)
    float total = 0.0f;
    for (int j = t; j < count; j += kUnitThreads) {
        const float e = exp_approx(__fadd_rn(sh.scores[j], -maximum));
        sh.scores[j] = e;
        total = __fadd_rn(total, e);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, d));
    if (lane == 0) sh.reduce[warp] = total;
    sync();
    total = sh.reduce[0];
#pragma unroll
    for (int i = 1; i < kUnitThreads / 32; ++i) total = __fadd_rn(total, sh.reduce[i]);

    // P.V, unnormalised
    const int slice = t >> 4, cg = t & 15;
    const uint16_t *vbase = v_head + (size_t)begin * key_stride + 8 * cg;
    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
    for (int j = slice; j < count; j += kUnitSlices) {
        const uint16_t *vr = vbase + (size_t)j * key_stride;
        if (FRESH && j == newest) vr = sh.fresh_v + 8 * cg;
        const uint4 v = *reinterpret_cast<const uint4 *>(vr);
        const float p = sh.scores[j];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[2 * i] = __fadd_rn(acc[2 * i], __fmul_rn(p, __uint_as_float(w[i] << 16)));
            acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], __fmul_rn(p, __uint_as_float(w[i] & 0xffff0000u)));
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sh.partial[slice][8 * cg + i] = acc[i];
    sync();
    float sum = 0.0f;
    if (t < kUnitHeadDim) {
        sum = sh.partial[0][t];
#pragma unroll
        for (int i = 1; i < kUnitSlices; ++i) sum = __fadd_rn(sum, sh.partial[i][t]);
    }

    if (splits > 1) {
        float *mine = scratch + ((size_t)unit * launched + split) * kUnitRecord;
        if (t < kUnitHeadDim) mine[t] = sum;
        if (t == 0) {
            mine[kUnitHeadDim] = maximum;
            mine[kUnitHeadDim + 1] = total;
        }
        __threadfence();
        sync();
        if (t == 0) {
            const uint32_t before = atomicAdd(counters + unit, 1u);
            sh.arrived = before;
            if (before == (uint32_t)splits - 1u) counters[unit] = 0u;  // the counter is zero again for the next launch
        }
        sync();
        if (sh.arrived != (uint32_t)splits - 1u) return false;
        __threadfence();
        if (t < kUnitHeadDim) {
            const float *all = scratch + (size_t)unit * launched * kUnitRecord;
            float top = -INFINITY;
            for (int s = 0; s < splits; ++s) top = fmaxf(top, __ldcg(all + s * kUnitRecord + kUnitHeadDim));
            sum = 0.0f;
            total = 0.0f;
            for (int s = 0; s < splits; ++s) {
                const float *rec = all + s * kUnitRecord;
                const float weight = exp_approx(__fadd_rn(__ldcg(rec + kUnitHeadDim), -top));  // 0 for an empty split
                total = __fadd_rn(total, __fmul_rn(__ldcg(rec + kUnitHeadDim + 1), weight));
                sum = __fadd_rn(sum, __fmul_rn(__ldcg(rec + t), weight));
            }
        }
    }
    if (t < kUnitHeadDim) {
        const float o = bf16_rne(__fdiv_rn(sum, total));
        T::store(out_head + t, o);
        if (maxima_row) {  // max |out| of the row, for a quantizer that takes its maximum from the producer
            const uint32_t m = warp_max_u32(absmax_key(o));
            if (lane == 0) atomicMax(maxima_row, m);
        }
    }
    return true;
}

}  // namespace w8a8
