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
//   * the keys of a row are split over up to 16 CTAs (one per 64 visible keys, at most 256 keys each) whose partial
//     (maximum, total, sums) the last CTA to arrive combines, so a short and a long sequence in the same batch both
//     spread over the GPU.  The number of splits is a function of the row's context length alone, never of the batch:
//     a sequence decoded alone and the same sequence decoded inside a batch produce the same bits.
// float32 sums are reassociated relative to the reference's one-thread-per-key kernel, and products are fused
// multiply-adds (q, k, v are bf16 values, so a product is exact either way and only the additions round); the result
// stays inside the reference's own bound for this operator (|err| <= 2e-4 + 1 % |x|, docs/qwen3-8b-w8a8/coverage.md:28).
#include "../../include/qwen3_glue.h"
#include "../../include/w8a8.h"
#include "common.cuh"
#include "internal.h"

namespace w8a8 {
namespace {

constexpr int kHeadDim = 128;
constexpr int kMaxContext = 4096;     // src/lib.rs:18
constexpr int kThreads = 256;
constexpr int kSlices = 16;           // key slices of the P.V product
constexpr int kMaxSplits = 16;        // CTAs per (row, key/value head group)
constexpr int kKeysPerSplit = 64;     // a split is not worth its combine step for fewer keys
constexpr int kMaxChunk = kMaxContext / kMaxSplits;  // keys per split at the longest context: 256
constexpr int kRecord = kHeadDim + 4;  // floats per (row, head, split) in the workspace: 128 sums, maximum, total, padding

__device__ __forceinline__ void record_range_fault(uint32_t *status, uint32_t detail) {
    if (status && atomicCAS(status, 0u, (uint32_t)FAULT_CACHE_RANGE) == 0u) status[1] = detail;
}

__device__ __forceinline__ float dot16_fma(const float (&qv)[16], const uint4 a, const uint4 b) {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        s = __fmaf_rn(qv[2 * i], __uint_as_float(w[i] << 16), s);
        s = __fmaf_rn(qv[2 * i + 1], __uint_as_float(w[i] & 0xffff0000u), s);
    }
    return s;
}

// Key range of one split.  `chunk` keys per split: a multiple of 32, at least 64 (but for the last split), at most 256.
struct SplitPlan {
    int splits, chunk;
};
__host__ __device__ __forceinline__ SplitPlan plan_splits(int end) {
    int splits = (end + kKeysPerSplit - 1) / kKeysPerSplit;
    if (splits > kMaxSplits) splits = kMaxSplits;
    const int chunk = (((end + splits - 1) / splits) + 31) & ~31;
    SplitPlan p;
    p.chunk = chunk;
    p.splits = (end + chunk - 1) / chunk;  // rounding the chunk up can empty the trailing splits: they are not used
    return p;
}

template <class T, int GH>
__global__ void __launch_bounds__(kThreads) attention_batched_kernel(const typename T::storage *__restrict__ q, int64_t ldq, int q_heads,
                                                                     int kv_heads, const uint16_t *__restrict__ k_cache,
                                                                     const uint16_t *__restrict__ v_cache, int64_t cache_stride,
                                                                     const uint32_t *__restrict__ positions,
                                                                     typename T::storage *__restrict__ out, int64_t ldo, int capacity,
                                                                     uint32_t *maxima, float *scratch, uint32_t *counters,
                                                                     uint32_t *status) {
    __shared__ float scores[GH][kMaxChunk];
    __shared__ float query[GH][kHeadDim];
    __shared__ float reduce[kThreads / 32][GH];
    __shared__ float partial[kSlices][GH][kHeadDim];
    __shared__ uint32_t arrived;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int group = q_heads / kv_heads, chunks = group / GH;
    const int row = blockIdx.x / (kv_heads * chunks);
    const int kv = (blockIdx.x / chunks) % kv_heads;
    const int head0 = kv * group + (blockIdx.x % chunks) * GH;
    const int split = blockIdx.y;
    // The position was uploaded by the host before the step began, so it does not depend on the preceding kernel: the key
    // range of this CTA is known before the dependency wait, and its cache lines are pulled towards L2 meanwhile.  The one
    // line the preceding kernel is still writing (the newest key) is simply fetched again by the loads below.
    const uint32_t end_u = positions[row] + 1u;
    if (end_u > (uint32_t)capacity) {  // every split of the row takes this branch: nobody waits for anybody
        if (t == 0 && split == 0) record_range_fault(status, end_u);
        return;
    }
    const int end = (int)end_u;
    const SplitPlan plan = plan_splits(end);
    if (split >= plan.splits) return;
    const int begin = split * plan.chunk, stop = min(end, begin + plan.chunk);
    const int count = stop - begin;  // 1 .. 256
    const size_t key_stride = (size_t)kv_heads * kHeadDim;
    const uint16_t *kc = k_cache + (size_t)row * cache_stride + (size_t)kv * kHeadDim;
    const uint16_t *vc = v_cache + (size_t)row * cache_stride + (size_t)kv * kHeadDim;
    for (int i = t; i < 2 * count; i += kThreads) {  // two 128-byte lines per key and per cache
        const size_t off = ((size_t)(begin + (i >> 1)) * key_stride) * sizeof(uint16_t) + (size_t)(i & 1) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(kc) + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(vc) + off));
    }
    dependency_wait();
    for (int i = t; i < GH * kHeadDim; i += kThreads)
        query[i / kHeadDim][i % kHeadDim] = T::load(q + (size_t)row * ldq + (size_t)head0 * kHeadDim + i);
    __syncthreads();

    // scores: eight lanes per key (16 channels each), four keys per warp and sweep
    const int sub = lane & 7, grp = lane >> 3;
    float maximum[GH];
    {
        float qv[GH][16];
#pragma unroll
        for (int h = 0; h < GH; ++h)
#pragma unroll
            for (int i = 0; i < 16; ++i) qv[h][i] = query[h][16 * sub + i];
        const uint16_t *kbase = kc + (size_t)begin * key_stride + 16 * sub;
#pragma unroll
        for (int h = 0; h < GH; ++h) maximum[h] = -INFINITY;
#pragma unroll 2
        for (int j0 = warp * 4; j0 < count; j0 += (kThreads / 32) * 4) {
            const int j = j0 + grp;
            uint4 a = make_uint4(0, 0, 0, 0), b = a;
            if (j < count) {
                const uint4 *kr = reinterpret_cast<const uint4 *>(kbase + (size_t)j * key_stride);
                a = kr[0];
                b = kr[1];
            }
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                float s = dot16_fma(qv[h], a, b);
                s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 4));
                s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
                s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
                s = __fmul_rn(s, 0.08838834764831845f);
                if (j < count) {
                    maximum[h] = fmaxf(maximum[h], s);
                    if (sub == 0) scores[h][j] = s;
                }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < GH; ++h) {
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) maximum[h] = fmaxf(maximum[h], __shfl_xor_sync(0xffffffffu, maximum[h], d));
        if (lane == 0) reduce[warp][h] = maximum[h];
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < GH; ++h) {
        maximum[h] = reduce[0][h];
#pragma unroll
        for (int i = 1; i < kThreads / 32; ++i) maximum[h] = fmaxf(maximum[h], reduce[i][h]);
    }
    __syncthreads();

    // softmax numerators (the reference's ex2.approx form) and their total; a split holds at most one key per thread
    float total[GH];
#pragma unroll
    for (int h = 0; h < GH; ++h) {
        float e = 0.0f;
        if (t < count) {
            e = exp_approx(__fadd_rn(scores[h][t], -maximum[h]));
            scores[h][t] = e;
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) e = __fadd_rn(e, __shfl_xor_sync(0xffffffffu, e, d));
        if (lane == 0) reduce[warp][h] = e;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < GH; ++h) {
        total[h] = reduce[0][h];
#pragma unroll
        for (int i = 1; i < kThreads / 32; ++i) total[h] = __fadd_rn(total[h], reduce[i][h]);
    }

    // P.V, unnormalised: sixteen key slices x sixteen lanes of 8 channels
    {
        const int slice = t >> 4, cg = t & 15;
        const uint16_t *vbase = vc + (size_t)begin * key_stride + 8 * cg;
        float acc[GH][8];
#pragma unroll
        for (int h = 0; h < GH; ++h)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[h][i] = 0.0f;
#pragma unroll 4
        for (int j = slice; j < count; j += kSlices) {
            const uint4 v = *reinterpret_cast<const uint4 *>(vbase + (size_t)j * key_stride);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int h = 0; h < GH; ++h) {
                const float p = scores[h][j];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[h][2 * i] = __fmaf_rn(p, __uint_as_float(w[i] << 16), acc[h][2 * i]);
                    acc[h][2 * i + 1] = __fmaf_rn(p, __uint_as_float(w[i] & 0xffff0000u), acc[h][2 * i + 1]);
                }
            }
        }
#pragma unroll
        for (int h = 0; h < GH; ++h)
#pragma unroll
            for (int i = 0; i < 8; ++i) partial[slice][h][8 * cg + i] = acc[h][i];
    }
    __syncthreads();

    const bool combine = plan.splits > 1;
    if (combine) {
        // leave (sums, maximum, total) of this split; the last split of the row's head group to arrive combines them
        for (int o = t; o < GH * kHeadDim; o += kThreads) {
            const int h = o / kHeadDim, c = o % kHeadDim;
            float sum = partial[0][h][c];
#pragma unroll
            for (int i = 1; i < kSlices; ++i) sum = __fadd_rn(sum, partial[i][h][c]);
            float *mine = scratch + (((size_t)row * q_heads + head0 + h) * kMaxSplits + split) * kRecord;
            mine[c] = sum;
            if (c == 0) {
                float mx = maximum[0], tot = total[0];
#pragma unroll
                for (int k = 1; k < GH; ++k)
                    if (h == k) {
                        mx = maximum[k];
                        tot = total[k];
                    }
                mine[kHeadDim] = mx;
                mine[kHeadDim + 1] = tot;
            }
        }
        __threadfence();
        __syncthreads();
        if (t == 0) {
            const uint32_t before = atomicAdd(counters + blockIdx.x, 1u);
            arrived = before;
            if (before == (uint32_t)plan.splits - 1u) counters[blockIdx.x] = 0u;  // zero again for the next launch
        }
        __syncthreads();
        if (arrived != (uint32_t)plan.splits - 1u) return;
        __threadfence();
    }
    for (int o = t; o < GH * kHeadDim; o += kThreads) {
        const int h = o / kHeadDim, c = o % kHeadDim;
        float sum, den;
        if (combine) {
            const float *all = scratch + ((size_t)row * q_heads + head0 + h) * kMaxSplits * kRecord;
            float top = -INFINITY;
            for (int s = 0; s < plan.splits; ++s) top = fmaxf(top, __ldcg(all + s * kRecord + kHeadDim));
            sum = 0.0f;
            den = 0.0f;
            for (int s = 0; s < plan.splits; ++s) {
                const float *rec = all + s * kRecord;
                const float weight = exp_approx(__fadd_rn(__ldcg(rec + kHeadDim), -top));
                den = __fmaf_rn(__ldcg(rec + kHeadDim + 1), weight, den);
                sum = __fmaf_rn(__ldcg(rec + c), weight, sum);
            }
        } else {
            sum = partial[0][h][c];
#pragma unroll
            for (int i = 1; i < kSlices; ++i) sum = __fadd_rn(sum, partial[i][h][c]);
            den = total[0];
#pragma unroll
            for (int k = 1; k < GH; ++k)
                if (h == k) den = total[k];
        }
        const float v = bf16_rne(__fdiv_rn(sum, den));
        T::store(out + (size_t)row * ldo + (size_t)(head0 + h) * kHeadDim + c, v);
        if (maxima) {  // max |out| of the row, for a quantizer that takes its maximum from the producer
            const uint32_t m = warp_max_u32(absmax_key(v));
            if (lane == 0) atomicMax(maxima + row, m);
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

size_t workspace_bytes(int rows, int q_heads, int kv_heads) {
    // arrival counters (one per CTA column of the launch, at most one per (row, head)), padded to 256 bytes, then the
    // partial results of every (row, head, split)
    const size_t counters = (((size_t)rows * q_heads * sizeof(uint32_t)) + 255) & ~(size_t)255;
    (void)kv_heads;
    return counters + (size_t)rows * q_heads * kMaxSplits * kRecord * sizeof(float);
}

template <class T, int GH>
cudaError_t launch_batched(const void *q, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache, const uint16_t *v_cache,
                           int64_t cache_stride, const uint32_t *positions, void *out, int64_t ldo, int capacity, uint32_t *maxima,
                           void *workspace, cudaStream_t s) {
    typedef typename T::storage S;
    const size_t counters = (((size_t)rows * q_heads * sizeof(uint32_t)) + 255) & ~(size_t)255;
    uint32_t *cnt = static_cast<uint32_t *>(workspace);
    float *scratch = reinterpret_cast<float *>(static_cast<char *>(workspace) + counters);
    const dim3 grid(rows * kv_heads * ((q_heads / kv_heads) / GH), kMaxSplits);
    return launch_kernel(attention_batched_kernel<T, GH>, grid, dim3(kThreads), (size_t)0, s, (const S *)q, ldq, q_heads, kv_heads, k_cache,
                         v_cache, cache_stride, positions, (S *)out, ldo, capacity, maxima, scratch, cnt, device_status_ptr());
}

template <class T>
cudaError_t launch_batched_any(const void *q, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                               const uint16_t *v_cache, int64_t cache_stride, const uint32_t *positions, void *out, int64_t ldo,
                               int capacity, uint32_t *maxima, void *workspace, cudaStream_t s) {
    const int group = q_heads / kv_heads;
    if (group % 4 == 0)
        return launch_batched<T, 4>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, cache_stride, positions, out, ldo, capacity, maxima, workspace, s);
    if (group % 2 == 0)
        return launch_batched<T, 2>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, cache_stride, positions, out, ldo, capacity, maxima, workspace, s);
    return launch_batched<T, 1>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, cache_stride, positions, out, ldo, capacity, maxima, workspace, s);
}

}  // namespace
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
    REQUIRE((long long)rows * q_heads <= 2147483647ll / 64, W8A8_ERR_UNSUPPORTED);
    cudaError_t e = dtype == W8A8_BF16
                        ? launch_batched_any<Bf16>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, cache_stride, positions, out, ldo,
                                                   capacity, maxima, workspace, (cudaStream_t)stream)
                        : launch_batched_any<F32>(q, ldq, rows, q_heads, kv_heads, k_cache, v_cache, cache_stride, positions, out, ldo,
                                                  capacity, maxima, workspace, (cudaStream_t)stream);
    return e == cudaSuccess ? W8A8_OK : fail_cuda(e, "batched attention launch");
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
