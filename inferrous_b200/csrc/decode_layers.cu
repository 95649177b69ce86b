// One decode step of a Qwen3 decoder stack (one token, one sequence) as ONE resident kernel: every layer's
// RMSNorm + quantize -> Q|K|V -> head norm + rotary + cache append -> attention -> quantize -> O + residual ->
// RMSNorm + quantize -> gate|up + SwiGLU -> quantize -> down + residual, with grid-wide barriers between the
// steps that depend on each other instead of kernel boundaries.
//
// Why: launched as separate kernels a step is ten dependent launches per layer, and at one token each of them is
// shorter than the latency of the dependency itself (the reference's answer to the same problem is its captured
// graph with programmatic edges and next-weight prefetch CTAs, src/graph.rs:63-127, src/kernels.rs:173-237).  Here
// one CTA per SM stays resident for the whole stack:
//   * the activation quantizers run as a prologue of the projection that consumes them, once per SM (not once per
//     launch-sized CTA);
//   * while thread 0 of a CTA polls a barrier, the other warps ask L2 for the first part of the CTA's share of the NEXT
//     matrix (weights are immutable), and inside a projection every warp keeps such requests one batch of rows ahead
//     of its loads, so the HBM stream does not stop dead at a barrier.  64 KiB per CTA and matrix is the measured
//     optimum: deeper requests cost more than they hide;
//   * head norm + rotary embedding are done by the attention units themselves (each recomputes its query head and,
//     where its key range holds the newest position, that key), which removes one dependent step per layer.
// Measured on a B200 (Qwen3-8B shapes, context 130..260): 58 us per layer, of which streaming the 193 MB of weights
// 28.6 us, the four quantizer prologues 9.2 us, attention about 8 us and the five barriers with the skew in front of
// them the rest; 2.13 ms per token against 2.47 ms for the same step as ten launches per layer.  Things that were tried
// and measured slower are noted where they would go (bulk L2 requests, more rows in flight per warp, the steps as
// separate non-inlined functions).
// Arithmetic: exactly that of the separate kernels (quantize.cu, gemv.cu, forward_glue.cu), so a step gives the
// same bits as the launch-per-operator path: int32 sums are exact, every float operation is element-wise or follows
// the same fixed association, and attention is the shared device function of attention_unit.cuh.
//
// Every wait is bounded (about two seconds): on expiry the waiter raises the abort word, records WAIT_GRID in the
// device status word, and every CTA leaves at its next barrier.  The kernel is launched cooperatively, so either all
// of its CTAs are resident or the launch fails; it never waits for a CTA that cannot run.
#include "../../include/qwen3_glue.h"
#include "../../include/w8a8.h"
#include "attention_unit.cuh"
#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"

#include <cstdlib>
#include <new>
#include <vector>

struct qwen3_decode_plan;

namespace w8a8 {
namespace {

constexpr int kThreads = 512;
constexpr int kGroupWarps = 8;              // a group of eight warps covers 4096 bytes of a weight row per load round
constexpr int kGroupBytes = kGroupWarps * 32 * 16;
constexpr int kMaxRounds = 3;               // K <= 12288
constexpr int kMaxK = kMaxRounds * kGroupBytes;
constexpr int kMaxCtaRows = 256;            // weight rows one CTA may own in a projection
constexpr int kHeadDim = kUnitHeadDim;

struct LayerDev {
    const void *norm1, *norm2;      // RMSNorm gains, carrier storage type
    const float *q_gain, *k_gain;   // head-norm gains
    const int8_t *qkv, *o, *gate, *up, *down;
    const float *qkv_s, *o_s, *gate_s, *up_s, *down_s;
    uint16_t *k_cache, *v_cache;    // [capacity][kv_heads][128] bf16
};

struct StepDev {
    const LayerDev *layers;
    int n_layers, hidden, q_heads, kv_heads, inter, capacity, splits;
    float eps;
    const float *rope;          // [capacity][128]: cos 0..63, sin 0..63
    const uint32_t *control;    // {token, position}
    void *hidden_io;            // [hidden]: embedding row in, last layer's output out
    void *residual;             // [hidden]
    void *qkv;                  // [(q_heads + 2 kv_heads) * 128]
    void *attn;                 // [q_heads * 128]
    void *act;                  // [inter]
    float *scratch;             // attention: per (head, split) records
    uint32_t *counters;         // attention: per head arrival counters (zero between launches)
    uint32_t *maxima;           // [layer][2]: max |v| of the attention row and of the SwiGLU row as absmax_key, zeroed with `sync`
    uint32_t *sync;             // {arrivals, abort}: zeroed by the host before every launch
    uint32_t *status;
    long long ahead_bytes;      // per CTA: bytes of the next matrix requested from L2 while waiting at the barrier in front of it
    long long ahead_more;       // per CTA: further bytes of gate and up requested one barrier earlier still (the O projection is short)
    int ahead_rows;             // inside a projection: L2 requests run this many row batches ahead of the loads
    long long *trace;           // optional: [CTA][layer][kTracePoints] SM cycle counts at the step boundaries of a layer
    // tensor parallel (decode_layers_tp_kernel): O and down own a slice of the input channels, their partial outputs are
    // summed over the ranks through packet buffers in peer memory
    uint2 *ll[kTpMaxRanks];     // packet buffer of every rank: [2 halves][tp sources][hidden] packets {value bits, tag}
    uint32_t *seq;              // local: [0] = exchanges completed by earlier steps (the tag base of this step)
    float *reduced;             // [hidden]: the summed row of an exchange, sliced form (below)
    int rank, tp, sliced;
};

// Points of a layer at which thread 0 of every CTA notes its SM's cycle counter when the plan carries a trace buffer.
enum TracePoint {
    TP_START = 0, TP_NORM1, TP_QKV, TP_ARRIVE1, TP_PASS1, TP_ATTENTION, TP_PASS2, TP_QUANT_O, TP_O, TP_PASS3, TP_NORM2, TP_GATE_UP,
    TP_PASS4, TP_QUANT_DOWN, TP_DOWN, TP_PASS5, kTracePoints
};

// ---- loads of values another CTA wrote during this kernel: from L2, never from this SM's L1 ----------------
template <class T> __device__ __forceinline__ void load_vec_cg(const typename T::storage *p, float (&v)[T::kVec]) {
    const uint4 r = __ldcg(reinterpret_cast<const uint4 *>(p));
    Vec<T>::unpack(r, v);
}
template <class T> __device__ __forceinline__ float load_one_cg(const typename T::storage *p);
template <> __device__ __forceinline__ float load_one_cg<Bf16>(const uint16_t *p) { return bf16_to_f32(__ldcg(p)); }
template <> __device__ __forceinline__ float load_one_cg<F32>(const float *p) { return __ldcg(p); }

// ---- grid-wide barrier ---------------------------------------------------------------------------------------
// sync[0] counts arrivals since the launch (the host zeroes it), so the n-th barrier of the step (n = 1, 2, ...) is
// passed when it reaches n * gridDim.x.  Returns false when the wait was abandoned; the caller leaves the kernel.
// `meanwhile(i, n)` is run by the other fifteen warps (thread i of n) after the CTA has arrived and while thread 0 polls:
// the L2 requests for the next matrix go there, off the path on which the other CTAs wait for this one.
template <class Meanwhile>
__device__ __forceinline__ bool grid_barrier(const StepDev &a, uint32_t ordinal, uint32_t *ok_smem, Meanwhile meanwhile) {
    __syncthreads();
    if (threadIdx.x >= 32) meanwhile((int)threadIdx.x - 32, kThreads - 32);
    if (threadIdx.x == 0) {
        const uint32_t target = ordinal * gridDim.x;
        // release: everything this CTA wrote (ordered before by the barrier above) is visible to whoever sees the count
        __threadfence();
        atomicAdd(a.sync, 1u);
        uint32_t good = 1;
        unsigned long long t0 = 0;
        for (uint32_t spin = 1;; ++spin) {
            uint32_t seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.sync) : "memory");
            if (seen >= target) break;
            if ((spin & 63u) == 0) {
                uint32_t stop;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(stop) : "l"(a.sync + 1) : "memory");
                if (stop) { good = 0; break; }
                const unsigned long long now = global_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > kWaitLimitNs) {
                    atomicExch(a.sync + 1, 1u);
                    if (a.status && atomicCAS(a.status, 0u, (uint32_t)WAIT_GRID) == 0u) a.status[1] = blockIdx.x;
                    good = 0;
                    break;
                }
            }
        }
        *ok_smem = good;
    }
    __syncthreads();
    return *ok_smem != 0;
}
// The barriers of layer l in step order: in front of Q|K|V (layers after the first), attention, O, gate|up, down.
enum { BAR_QKV = 0, BAR_ATTENTION = 1, BAR_O = 2, BAR_GATE_UP = 3, BAR_DOWN = 4, kBarriersPerLayer = 5 };
__device__ __forceinline__ uint32_t barrier_ordinal(int l, int which) { return (uint32_t)(l * kBarriersPerLayer + which); }

// This CTA's rows [r0, r1) of an N-row matrix.
__device__ __forceinline__ void cta_rows(int N, int &r0, int &r1) {
    r0 = (int)(((long long)N * blockIdx.x) / gridDim.x);
    r1 = (int)(((long long)N * (blockIdx.x + 1)) / gridDim.x);
}

// Ask L2 for bytes [from, to) of this CTA's rows of an [N][K] matrix, one 128-byte line per prefetch instruction, thread
// i of n.  (Bulk requests of 16 KiB per instruction, cp.async.bulk.prefetch.L2, are cheaper to issue and were measured
// slower overall: 2.53 against 2.44 ms per token.)
__device__ __forceinline__ void request_rows(const int8_t *w, int K, int N, long long from, long long to, int i, int n) {
    int r0, r1;
    cta_rows(N, r0, r1);
    const long long share = (long long)(r1 - r0) * K;
    if (to > share) to = share;
    if (to <= from) return;
    const unsigned long long base = reinterpret_cast<unsigned long long>(w) + (unsigned long long)r0 * K;
    const unsigned long long begin = (base + (unsigned long long)from + 127ull) & ~127ull, end = (base + (unsigned long long)to) & ~127ull;
    for (unsigned long long p = begin + 128ull * i; p < end; p += 128ull * n) asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// ---- quantizing prologues: the unquantized row -> int8 codes in shared memory, returns the scale --------------
struct PrologueShared {
    float red[256];
    uint32_t slots[32];
};

// quantize (src/kernels.rs:415-452): m = max(1e-8, max|x|) ignoring NaN; s = m / 127; q = rne(clamp(x / s))
template <class T>
__device__ __forceinline__ float prologue_plain(const typename T::storage *x, int K, int8_t *sq, float *row, PrologueShared &ps, int tid) {
    constexpr int V = T::kVec;
    float m = 1e-8f;
    for (int j = tid * V; j < K; j += kThreads * V) {
        float v[V];
        load_vec_cg<T>(x + j, v);
#pragma unroll
        for (int i = 0; i < V; ++i) m = fmaxf(m, fabsf(v[i]));  // fmaxf drops a NaN operand
#pragma unroll
        for (int i = 0; i < V; i += 4) *reinterpret_cast<float4 *>(row + j + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    const float s = __fdiv_rn(block_max(m, ps.slots, tid), 127.0f);
    const float inv = __frcp_rn(s);
    for (int j = tid * V; j < K; j += kThreads * V) {  // each thread re-reads exactly the elements it parked
        int c[V];
#pragma unroll
        for (int i = 0; i < V; ++i) c[i] = quant_code(row[j + i], s, inv);
        store_codes<V>(sq + j, c);
    }
    return s;
}

// quantize() of a row whose producers left max |x| in `*published` (absmax_key; quantize_with_max, src/kernels.rs:
// 134-172): one pass, nothing parked in shared memory and no block-wide reduction.
template <class T>
__device__ __forceinline__ float prologue_published(const typename T::storage *x, int K, const uint32_t *published, int8_t *sq, int tid) {
    constexpr int V = T::kVec;
    const float m = fmaxf(1e-8f, __uint_as_float(__ldcg(published)));
    const float s = __fdiv_rn(m, 127.0f);
    const float inv = __frcp_rn(s);
    for (int j = tid * V; j < K; j += kThreads * V) {
        float v[V];
        load_vec_cg<T>(x + j, v);
        int c[V];
#pragma unroll
        for (int i = 0; i < V; ++i) c[i] = quant_code(v[i], s, inv);
        store_codes<V>(sq + j, c);
    }
    return s;
}

// norm_quantize (src/kernels.rs:479-576): the reference's summation tree (256 strided partial sums, distances
// 128..1), y = bf16((x * rsqrt(mean + eps)) * gain), m = max(1e-8, max|y|), s = m / 127
// The part of norm_quantize behind the load: `row` holds the K values of x.
template <class T>
__device__ __forceinline__ float rmsnorm_row(const typename T::storage *gain, float eps, int K, int8_t *sq, float *row,
                                             PrologueShared &ps, int tid) {
    constexpr int V = T::kVec;
    if (tid < 256) {
        float p = 0.0f;
        for (int j = tid; j < K; j += 256) p = __fadd_rn(p, __fmul_rn(row[j], row[j]));
        ps.red[tid] = p;
    }
    __syncthreads();
    if (tid < 32) {
        const float *red = ps.red;
        float t = __fadd_rn(__fadd_rn(__fadd_rn(red[tid], red[tid + 128]), __fadd_rn(red[tid + 64], red[tid + 192])),
                            __fadd_rn(__fadd_rn(red[tid + 32], red[tid + 160]), __fadd_rn(red[tid + 96], red[tid + 224])));
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, d));
        if (tid == 0) ps.red[0] = t;
    }
    __syncthreads();
    const float inv_norm = rsqrt_approx(__fadd_rn(__fdiv_rn(ps.red[0], (float)K), eps));
    float m = 1e-8f;
    for (int j = tid * V; j < K; j += kThreads * V) {
        float g[V];
        Vec<T>::load(gain + j, g);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float y = bf16_rne(__fmul_rn(__fmul_rn(row[j + i], inv_norm), g[i]));
            m = fmaxf(m, fabsf(y));
            row[j + i] = y;
        }
    }
    const float s = __fdiv_rn(block_max(m, ps.slots, tid), 127.0f);
    const float inv = __frcp_rn(s);
    for (int j = tid * V; j < K; j += kThreads * V) {
        int c[V];
#pragma unroll
        for (int i = 0; i < V; ++i) c[i] = quant_code(row[j + i], s, inv);
        store_codes<V>(sq + j, c);
    }
    return s;
}

// norm_quantize (src/kernels.rs:479-576): the reference's summation tree (256 strided partial sums, distances
// 128..1), y = bf16((x * rsqrt(mean + eps)) * gain), m = max(1e-8, max|y|), s = m / 127
template <class T>
__device__ __forceinline__ float prologue_rmsnorm(const typename T::storage *x, const typename T::storage *gain, float eps, int K,
                                                  int8_t *sq, float *row, PrologueShared &ps, int tid) {
    constexpr int V = T::kVec;
    for (int j = tid * V; j < K; j += kThreads * V) {
        float v[V];
        load_vec_cg<T>(x + j, v);
#pragma unroll
        for (int i = 0; i < V; i += 4) *reinterpret_cast<float4 *>(row + j + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
    __syncthreads();
    return rmsnorm_row<T>(gain, eps, K, sq, row, ps, tid);
}

// ---- one projection, this CTA's share ------------------------------------------------------------------------
// The CTA owns the weight rows [r0, r1) (row pairs (gate c, up c) for the SwiGLU form).  Its sixteen warps form two
// groups of eight; a group takes every other row and spreads the row's K bytes over its 256 lanes, 16 bytes each per
// round of 4096 bytes, so the lane's slice of the activation codes stays in registers for the whole projection.
// Per row and warp: J loads, 4 J dp4a, one warp-wide integer add; the eight partial sums of a row meet in shared
// memory and one thread per row finishes it (exact: int32).
enum { PRJ_PLAIN = 0, PRJ_RESIDUAL = 1, PRJ_SWIGLU = 2, PRJ_PUSH = 3 };

// Tensor parallel: one 8-byte packet {value bits, tag of the exchange} to the same slot of every rank (plain peer stores
// over NVLink); value and tag travel in one store, so the reader needs no fence, only to see the tag.
__device__ __forceinline__ void push_packet(const StepDev &a, uint32_t exchange, uint32_t tag, int element, float value) {
    const size_t at = ((size_t)(exchange & 1u) * a.tp + a.rank) * a.hidden + element;
    const uint32_t bits = __float_as_uint(value);
    for (int p = 0; p < a.tp; ++p)
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(a.ll[p] + at), "r"(bits), "r"(tag) : "memory");
}

__device__ __forceinline__ int dp4a_16(const uint4 &w, const uint4 &x, int acc) {
    acc = __dp4a((int)w.x, (int)x.x, acc);
    acc = __dp4a((int)w.y, (int)x.y, acc);
    acc = __dp4a((int)w.z, (int)x.z, acc);
    acc = __dp4a((int)w.w, (int)x.w, acc);
    return acc;
}

template <class T, int EPI, int J>
__device__ void project(const StepDev &a, const int8_t *__restrict__ w0, const int8_t *__restrict__ w1,
                        const float *__restrict__ ws0, const float *__restrict__ ws1, int N, int K, float a_scale,
                        const int8_t *sq, int *red, const typename T::storage *residual, typename T::storage *out, int tid,
                        uint32_t exchange = 0, uint32_t tag = 0, uint32_t *maxima = nullptr) {
    constexpr int R = (EPI == PRJ_SWIGLU) ? 2 : 1;
    // row units per batch: eight 16-byte loads in flight per lane.  Twelve or sixteen fit the registers too and were
    // measured 5-10 % slower per token.
    constexpr int U = (R * J == 1) ? 8 : (R * J == 2) ? 4 : (R * J == 3) ? 3 : (R * J == 4) ? 2 : 1;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = warp / kGroupWarps, slot = warp % kGroupWarps;
    int r0, r1;
    cta_rows(N, r0, r1);
    const int units = r1 - r0;
    const int mine = (units - g + 1) / 2;  // this group's units: local index g, g + 2, ...

    // what the finishing thread of a row needs, requested now so that the end of the projection waits on registers
    float pre_s0 = 0.0f, pre_s1 = 0.0f, pre_res = 0.0f;
    if (tid < units) {
        pre_s0 = ws0[r0 + tid];
        if (EPI == PRJ_SWIGLU) pre_s1 = ws1[r0 + tid];
        if (EPI == PRJ_RESIDUAL) pre_res = load_one_cg<T>(residual + r0 + tid);
    }

    int off[J];
    bool valid[J];
    uint4 av[J];
#pragma unroll
    for (int j = 0; j < J; ++j) {
        off[j] = j * kGroupBytes + slot * 512 + lane * 16;
        valid[j] = off[j] < K;
        av[j] = valid[j] ? *reinterpret_cast<const uint4 *>(sq + off[j]) : make_uint4(0, 0, 0, 0);
    }

    uint4 wv[U][R][J];
    auto issue = [&](int first) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = first + u;
            const bool live = idx < mine;
            const long long row = (long long)(r0 + g + 2 * idx) * K;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int8_t *wr = (r == 0 ? w0 : w1) + row;
#pragma unroll
                for (int j = 0; j < J; ++j) wv[u][r][j] = (live && valid[j]) ? ld_stream_16(wr + off[j]) : make_uint4(0, 0, 0, 0);
            }
            // L2 requests a fixed number of batches ahead of the loads (one lane per 128-byte line)
            const int far = idx + a.ahead_rows * U;
            if (a.ahead_rows > 0 && far < mine && (lane & 7) == 0) {
                const long long frow = (long long)(r0 + g + 2 * far) * K;
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int j = 0; j < J; ++j)
                        if (valid[j]) asm volatile("prefetch.global.L2 [%0];" ::"l"((r == 0 ? w0 : w1) + frow + off[j]));
            }
        }
    };
    issue(0);
    for (int first = 0; first < mine; first += U) {
        int acc[U][R];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int r = 0; r < R; ++r) {
                int s = 0;
#pragma unroll
                for (int j = 0; j < J; ++j) s = dp4a_16(wv[u][r][j], av[j], s);
                acc[u][r] = s;
            }
        if (first + U < mine) issue(first + U);
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int total = warp_sum_i32(acc[u][r]);
                const int idx = first + u;
                if (lane == 0 && idx < mine) red[((g + 2 * idx) * R + r) * kGroupWarps + slot] = total;
            }
    }
    __syncthreads();
    uint32_t key = 0;  // PRJ_SWIGLU with `maxima`: max |value| of the rows this thread finished
    if (tid < units) {
        int sum[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int4 lo = *reinterpret_cast<const int4 *>(red + (tid * R + r) * kGroupWarps);
            const int4 hi = *reinterpret_cast<const int4 *>(red + (tid * R + r) * kGroupWarps + 4);
            sum[r] = lo.x + lo.y + lo.z + lo.w + hi.x + hi.y + hi.z + hi.w;
        }
        const int c = r0 + tid;
        if (EPI == PRJ_SWIGLU) {
            const float gv = dequant(sum[0], a_scale, pre_s0);
            const float uv = dequant(sum[R - 1], a_scale, pre_s1);
            const float value = swiglu_value(gv, uv);
            T::store(out + c, value);
            key = absmax_key(value);
        } else if (EPI == PRJ_PUSH) {
            push_packet(a, exchange, tag, c, dequant(sum[0], a_scale, pre_s0));
        } else if (EPI == PRJ_RESIDUAL) {
            T::store(out + c, bf16_rne(__fadd_rn(pre_res, dequant(sum[0], a_scale, pre_s0))));
        } else {
            T::store(out + c, dequant(sum[0], a_scale, pre_s0));
        }
    }
    if (EPI == PRJ_SWIGLU && maxima) {  // the quantizer in front of `down` takes the row's maximum from here
        key = warp_max_u32(key);
        if (lane == 0 && key) atomicMax(maxima, key);
    }
}

template <class T, int EPI>
__device__ __forceinline__ void project_any(const StepDev &a, const int8_t *w0, const int8_t *w1, const float *ws0, const float *ws1,
                                            int N, int K, float a_scale, const int8_t *sq, int *red,
                                            const typename T::storage *residual, typename T::storage *out, int tid,
                                            uint32_t exchange = 0, uint32_t tag = 0, uint32_t *maxima = nullptr) {
    if (K <= kGroupBytes) project<T, EPI, 1>(a, w0, w1, ws0, ws1, N, K, a_scale, sq, red, residual, out, tid, exchange, tag, maxima);
    else if (K <= 2 * kGroupBytes) project<T, EPI, 2>(a, w0, w1, ws0, ws1, N, K, a_scale, sq, red, residual, out, tid, exchange, tag, maxima);
    else project<T, EPI, 3>(a, w0, w1, ws0, ws1, N, K, a_scale, sq, red, residual, out, tid, exchange, tag, maxima);
}

// ---- attention: two units side by side per CTA ------------------------------------------------------------------
// Head RMSNorm + rotary embedding of one 128-wide head by one warp (prepare_qk, src/kernels.rs:1350-1443): lane l
// holds elements l, l+32, l+64, l+96, so the first tree level ((p[t] + p[t+64]) + (p[t+32] + p[t+96]) for t < 32) and
// the rotary pairs (t, t+64) are lane-local.
template <class T>
__device__ __forceinline__ void head_norm_rope(const typename T::storage *x, const float *gain, const float *trow, int lane,
                                               float (&r)[4]) {
    float v[4], g[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = load_one_cg<T>(x + lane + 32 * i);
        g[i] = gain[lane + 32 * i];
    }
    const float c0 = trow[lane], c1 = trow[lane + 32], s0 = trow[lane + 64], s1 = trow[lane + 96];
    float sum = __fadd_rn(__fadd_rn(__fmul_rn(v[0], v[0]), __fmul_rn(v[2], v[2])),
                          __fadd_rn(__fmul_rn(v[1], v[1]), __fmul_rn(v[3], v[3])));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, d));
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float inv = rsqrt_approx(__fadd_rn(__fdiv_rn(sum, 128.0f), 1e-6f));
    float n[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) n[i] = bf16_rne(__fmul_rn(__fmul_rn(v[i], inv), g[i]));
    r[0] = bf16_rne(__fadd_rn(__fmul_rn(n[0], c0), -__fmul_rn(n[2], s0)));
    r[2] = bf16_rne(__fadd_rn(__fmul_rn(n[2], c0), __fmul_rn(n[0], s0)));
    r[1] = bf16_rne(__fadd_rn(__fmul_rn(n[1], c1), -__fmul_rn(n[3], s1)));
    r[3] = bf16_rne(__fadd_rn(__fmul_rn(n[3], c1), __fmul_rn(n[1], s1)));
}

// Unit u of the step: split-major, so that the splits a short context leaves unused are the last units.
__device__ __forceinline__ void unit_of(const StepDev &a, int u, int &head, int &split) {
    split = u / a.q_heads;
    head = u % a.q_heads;
}

// Before the barrier in front of the attention step: ask L2 for the cache lines of this half-CTA's first unit.
__device__ __forceinline__ void request_cache(const StepDev &a, const LayerDev &L, int end, int i, int n) {
    const int half = i >= n / 2, t = half ? i - n / 2 : i, per_half = n / 2;
    const int u = blockIdx.x * 2 + half;
    if (u >= a.q_heads * a.splits) return;
    int head, split, splits, begin, stop;
    unit_of(a, u, head, split);
    unit_range(end, a.splits, split, splits, begin, stop);
    if (split >= splits) return;
    const int kv = head / (a.q_heads / a.kv_heads);
    const size_t stride_bytes = (size_t)a.kv_heads * kHeadDim * sizeof(uint16_t);
    const char *kline = reinterpret_cast<const char *>(L.k_cache) + (size_t)kv * kHeadDim * sizeof(uint16_t);
    const char *vline = reinterpret_cast<const char *>(L.v_cache) + (size_t)kv * kHeadDim * sizeof(uint16_t);
    for (int line = t; line < 2 * (stop - begin); line += per_half) {  // two 128-byte lines per key and per cache
        const size_t off = (size_t)(begin + (line >> 1)) * stride_bytes + (size_t)(line & 1) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(kline + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(vline + off));
    }
}

// Shared-memory copy of the keys and values of one unit (at most kStageKeys of them: contexts up to 9 x 64 keys).
constexpr int kStageKeys = 64;
struct UnitStage {
    uint16_t k[kStageKeys][kHeadDim];
    uint16_t v[kStageKeys][kHeadDim];
};
__device__ __forceinline__ bool unit_staged(int begin, int stop) { return stop - begin <= kStageKeys; }

// Before the barrier in front of the attention step: start the asynchronous copies of the cached keys and values of
// this half-CTA's first unit into shared memory (they were final before the launch; the key and value of this step's
// token are not among them), so that they arrive while the CTA waits for the others.  A unit of more than kStageKeys
// keys only gets its cache lines requested into L2.
__device__ __forceinline__ void stage_cache(const StepDev &a, const LayerDev &L, UnitStage *both, int end, int i) {
    // thread i + 32 of the CTA: the copies of a unit are started by threads of that unit's half, which wait for them
    const int tid = i + 32, half = tid >> 8, t = half ? tid - kUnitThreads : i, per_half = half ? kUnitThreads : kUnitThreads - 32;
    const int u = blockIdx.x * 2 + half;
    if (u >= a.q_heads * a.splits) return;
    int head, split, splits, begin, stop;
    unit_of(a, u, head, split);
    unit_range(end, a.splits, split, splits, begin, stop);
    if (split >= splits) return;
    const int kv = head / (a.q_heads / a.kv_heads);
    const size_t key_stride = (size_t)a.kv_heads * kHeadDim;
    const uint16_t *ks = L.k_cache + (size_t)kv * kHeadDim + (size_t)begin * key_stride;
    const uint16_t *vs = L.v_cache + (size_t)kv * kHeadDim + (size_t)begin * key_stride;
    if (!unit_staged(begin, stop)) {
        for (int line = t; line < 2 * (stop - begin); line += per_half) {  // two 128-byte lines per key and per cache
            const size_t off = (size_t)(line >> 1) * key_stride + (size_t)(line & 1) * 64;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(ks + off));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(vs + off));
        }
        return;
    }
    const int cached = min(stop, end - 1) - begin;  // key end - 1 is written during this step
    for (int c = t; c < cached * (kHeadDim / 8); c += per_half) {  // 16-byte pieces, sixteen per key
        const int key = c >> 4, piece = c & 15;
        const uint32_t kd = (uint32_t)__cvta_generic_to_shared(&both[half].k[key][8 * piece]);
        const uint32_t vd = (uint32_t)__cvta_generic_to_shared(&both[half].v[key][8 * piece]);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kd), "l"(ks + (size_t)key * key_stride + 8 * piece) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vd), "l"(vs + (size_t)key * key_stride + 8 * piece) : "memory");
    }
}

template <class T>
__device__ void attention_phase(const StepDev &a, const LayerDev &L, UnitShared *both, UnitStage *stage, int end, int tid,
                                uint32_t *maxima_row) {
    typedef typename T::storage S;
    const int half = tid >> 8, t = tid & 255, warp = t >> 5, lane = t & 31;
    UnitShared &sh = both[half];
    const SyncNamed sync{1 + half};
    const int group = a.q_heads / a.kv_heads;
    const size_t key_stride = (size_t)a.kv_heads * kHeadDim;
    const S *qkv = static_cast<const S *>(a.qkv);
    const float *trow = a.rope + (size_t)(end - 1) * kHeadDim;
    for (int u = blockIdx.x * 2 + half; u < a.q_heads * a.splits; u += 2 * gridDim.x) {
        int head, split, splits, begin, stop;
        unit_of(a, u, head, split);
        unit_range(end, a.splits, split, splits, begin, stop);
        if (split >= splits) continue;  // the same for all 256 threads
        const int kv = head / group;
        const bool holds_newest = begin <= end - 1 && end - 1 < stop;
        if (warp == 0) {
            float r[4];
            head_norm_rope<T>(qkv + (size_t)head * kHeadDim, L.q_gain, trow, lane, r);
#pragma unroll
            for (int i = 0; i < 4; ++i) sh.query[lane + 32 * i] = r[i];
        } else if (warp == 1 && holds_newest) {
            // the newest key and value are not in the cache yet: this unit makes its own copy, and the first query
            // head of the group also appends them to the cache (cache, src/kernels.rs:1470-1488)
            float r[4];
            head_norm_rope<T>(qkv + (size_t)(a.q_heads + kv) * kHeadDim, L.k_gain, trow, lane, r);
            const S *vx = qkv + (size_t)(a.q_heads + a.kv_heads + kv) * kHeadDim;
            const size_t at = ((size_t)(end - 1) * a.kv_heads + kv) * kHeadDim;
            const bool append = head % group == 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint16_t kb = (uint16_t)(__float_as_uint(r[i]) >> 16);
                const uint16_t vb = (uint16_t)(__float_as_uint(load_one_cg<T>(vx + lane + 32 * i)) >> 16);
                sh.fresh_k[lane + 32 * i] = kb;
                sh.fresh_v[lane + 32 * i] = vb;
                if (append) {
                    L.k_cache[at + lane + 32 * i] = kb;
                    L.v_cache[at + lane + 32 * i] = vb;
                }
            }
        }
        // the first unit of the half reads the copies that stage_cache started (`stage`: null where nothing was staged)
        const bool staged = stage && u < 2 * (int)gridDim.x && unit_staged(begin, stop);
        if (staged) asm volatile("cp.async.wait_all;" ::: "memory");
        sync();
        const uint16_t *keys = staged ? &stage[half].k[0][0] - (size_t)begin * kHeadDim : L.k_cache + (size_t)kv * kHeadDim;
        const uint16_t *values = staged ? &stage[half].v[0][0] - (size_t)begin * kHeadDim : L.v_cache + (size_t)kv * kHeadDim;
        attention_unit<T, true>(sh, sync, t, keys, values, staged ? (size_t)kHeadDim : key_stride, end,
                                splits, split, begin, stop, a.splits, head, a.scratch, a.counters,
                                static_cast<S *>(a.attn) + (size_t)head * kHeadDim, maxima_row);
        sync();  // sh is reused by this half's next unit
    }
}

// ---- the step -------------------------------------------------------------------------------------------------
template <bool STAGE> struct AttentionShared {
    UnitShared units[2];
    UnitStage stage[2];  // behind `row` in the union below: filled while the barrier after the Q|K|V step is waited for
};
template <> struct AttentionShared<false> {
    UnitShared units[2];
};
template <bool STAGE> struct StepSharedOf {
    int8_t codes[kMaxK];                       // the quantized activation row of the current projection
    int red[kMaxCtaRows * kGroupWarps];        // per weight row: the eight partial sums of its group
    PrologueShared ps;
    uint32_t ok;
    uint32_t pad[3];
    union {
        float row[kMaxK];                      // prologues: the unquantized / normalised row
        AttentionShared<STAGE> att;
    };
};
typedef StepSharedOf<true> StepShared;
static_assert(sizeof(StepShared) <= 227 * 1024, "shared memory of the decode kernel");

// The five steps of a layer are inlined into the layer loop on purpose: as separate (not inlined) functions each call
// spilled the registers that live across it, inside the streaming loops too, and a token took 4.9 ms instead of 2.2.
template <class T, bool TRACE>
__global__ void __launch_bounds__(kThreads, 1) decode_layers_kernel(const StepDev a) {
    typedef typename T::storage S;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    StepShared &sh = *reinterpret_cast<StepShared *>(smem_raw);
    const int tid = threadIdx.x;
    const uint32_t pos = a.control[1];
    if (pos >= (uint32_t)a.capacity) {  // every CTA takes this branch: nobody waits for anybody
        if (blockIdx.x == 0 && tid == 0 && a.status && atomicCAS(a.status, 0u, (uint32_t)FAULT_CACHE_RANGE) == 0u) a.status[1] = pos;
        return;
    }
    const int end = (int)pos + 1;
    const int q_width = a.q_heads * kHeadDim, qkv_width = (a.q_heads + 2 * a.kv_heads) * kHeadDim;
    S *hidden = static_cast<S *>(a.hidden_io), *residual = static_cast<S *>(a.residual);
    // TRACE is a separate instantiation: the marks cost 1 % of the step even when nothing is recorded
    long long *trace = TRACE && a.trace && tid == 0 ? a.trace + (size_t)blockIdx.x * a.n_layers * kTracePoints : nullptr;
    for (int l = 0; l < a.n_layers; ++l) {
        const LayerDev L = a.layers[l];  // all seventeen pointers at once: fetched one by one where they are used, each costs an L2 round trip on the critical path
        auto mark = [&](int point) {
            if (TRACE && trace) trace[l * kTracePoints + point] = clock64();
        };
        mark(TP_START);
        // norm1 + quantize -> Q|K|V
        float s = prologue_rmsnorm<T>(hidden, static_cast<const S *>(L.norm1), a.eps, a.hidden, sh.codes, sh.row, sh.ps, tid);
        __syncthreads();
        mark(TP_NORM1);
        project_any<T, PRJ_PLAIN>(a, L.qkv, nullptr, L.qkv_s, nullptr, qkv_width, a.hidden, s, sh.codes, sh.red, nullptr,
                                  static_cast<S *>(a.qkv), tid);
        mark(TP_QKV);
        mark(TP_ARRIVE1);
        if (!grid_barrier(a, barrier_ordinal(l, BAR_ATTENTION), &sh.ok, [&](int i, int n) {
                stage_cache(a, L, sh.att.stage, end, i);
                request_rows(L.o, q_width, a.hidden, 0, 1ll << 40, i, n);  // attention leaves HBM idle: the whole share of O
            }))
            return;
        mark(TP_PASS1);

        attention_phase<T>(a, L, sh.att.units, sh.att.stage, end, tid, a.maxima + 2 * l);
        mark(TP_ATTENTION);
        if (!grid_barrier(a, barrier_ordinal(l, BAR_O), &sh.ok, [&](int i, int n) {
                request_rows(L.gate, a.hidden, a.inter, 0, a.ahead_bytes, i, n);
                request_rows(L.up, a.hidden, a.inter, 0, a.ahead_bytes, i, n);
            }))
            return;
        mark(TP_PASS2);

        // quantize(attention row) -> O + residual
        s = prologue_published<T>(static_cast<const S *>(a.attn), q_width, a.maxima + 2 * l, sh.codes, tid);
        __syncthreads();
        mark(TP_QUANT_O);
        project_any<T, PRJ_RESIDUAL>(a, L.o, nullptr, L.o_s, nullptr, a.hidden, q_width, s, sh.codes, sh.red, hidden, residual, tid);
        mark(TP_O);
        if (!grid_barrier(a, barrier_ordinal(l, BAR_GATE_UP), &sh.ok, [&](int i, int n) {
                request_rows(L.gate, a.hidden, a.inter, a.ahead_bytes, a.ahead_bytes + a.ahead_more, i, n);
                request_rows(L.up, a.hidden, a.inter, a.ahead_bytes, a.ahead_bytes + a.ahead_more, i, n);
            }))
            return;
        mark(TP_PASS3);

        // norm2 + quantize -> gate|up + SwiGLU
        s = prologue_rmsnorm<T>(residual, static_cast<const S *>(L.norm2), a.eps, a.hidden, sh.codes, sh.row, sh.ps, tid);
        __syncthreads();
        mark(TP_NORM2);
        project_any<T, PRJ_SWIGLU>(a, L.gate, L.up, L.gate_s, L.up_s, a.inter, a.hidden, s, sh.codes, sh.red, nullptr,
                                   static_cast<S *>(a.act), tid, 0, 0, a.maxima + 2 * l + 1);
        mark(TP_GATE_UP);
        if (!grid_barrier(a, barrier_ordinal(l, BAR_DOWN), &sh.ok,
                          [&](int i, int n) { request_rows(L.down, a.inter, a.hidden, 0, a.ahead_bytes, i, n); }))
            return;
        mark(TP_PASS4);

        // quantize(act) -> down + residual
        s = prologue_published<T>(static_cast<const S *>(a.act), a.inter, a.maxima + 2 * l + 1, sh.codes, tid);
        __syncthreads();
        mark(TP_QUANT_DOWN);
        project_any<T, PRJ_RESIDUAL>(a, L.down, nullptr, L.down_s, nullptr, a.hidden, a.inter, s, sh.codes, sh.red, residual, hidden, tid);
        mark(TP_DOWN);
        if (l + 1 < a.n_layers) {
            const int8_t *next = a.layers[l + 1].qkv;
            if (!grid_barrier(a, barrier_ordinal(l + 1, BAR_QKV), &sh.ok,
                              [&](int i, int n) { request_rows(next, a.hidden, qkv_width, 0, a.ahead_bytes, i, n); }))
                return;
        }
        mark(TP_PASS5);
    }
}


// ---- the step under tensor parallelism ------------------------------------------------------------------------------
// Every rank runs this kernel on its shard (its query / key / value heads, its gate / up channels, its slice of the
// input channels of O and down).  The residual stream is replicated: every CTA of every rank keeps the whole hidden
// row and the whole residual row in its shared memory.  O and down send their partial outputs to every rank as tagged
// packets; the wait for the packets of an exchange takes the place of the grid-wide barrier behind those projections,
// and the reduction (sum in rank order in float32, bf16, + residual, bf16: what tp_reduce_kernel computes after
// w8a8_linear_allreduce) is the first part of the prologue that follows.  Two packet-buffer halves alternate; a rank
// can only run two exchanges ahead of another once that one has read the older half.
struct StepSharedTp {
    StepSharedOf<false> base;  // the two rows below leave no room for staged keys and values
    float hidden[kMaxK];    // the hidden row (the layer's input), every CTA its own copy
    float residual[kMaxK];  // hidden + attention block
};
static_assert(sizeof(StepSharedTp) <= 227 * 1024, "shared memory of the tensor-parallel decode kernel");

// Waits (bounded) for the packets of `exchange` from every rank and leaves out[e] = bf16(in[e] + bf16(sum_r y_r[e])).
// Thread t owns elements t, t + 512, ...; its packets (element-major, rank fastest) are taken sixteen at a time: all that
// are still missing are requested together, again and again until every tag is the exchange's, so the wait costs the
// time the last packet needs to arrive plus one round trip, not one round trip per packet.
__device__ __forceinline__ bool gather_exchange(const StepDev &a, uint32_t exchange, uint32_t tag, const float *in, float *out,
                                                uint32_t *ok_smem, int tid) {
    const uint2 *base = a.ll[a.rank] + (size_t)(exchange & 1u) * a.tp * a.hidden;
    constexpr int kBatch = 16;
    const int packets = ((a.hidden + kThreads - 1) / kThreads) * a.tp;
    bool good = true;
    float sum = 0.0f;
    for (int first = 0; first < packets && good; first += kBatch) {
        uint2 v[kBatch];
        uint32_t missing = 0;
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int idx = first + b, k = idx / a.tp;
            if (idx < packets && tid + k * kThreads < a.hidden) missing |= 1u << b;
        }
        unsigned long long t0 = 0;
        for (uint32_t spin = 1; missing; ++spin) {
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int idx = first + b, k = idx / a.tp, r = idx - k * a.tp, e = tid + k * kThreads;
                if (missing >> b & 1u)
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];"
                                 : "=r"(v[b].x), "=r"(v[b].y)
                                 : "l"(base + (size_t)r * a.hidden + e)
                                 : "memory");
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b)
                if ((missing >> b & 1u) && v[b].y == tag) missing &= ~(1u << b);
            if (missing && (spin & 63u) == 0) {
                uint32_t stop;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(stop) : "l"(a.sync + 1) : "memory");
                const unsigned long long now = global_ns();
                if (t0 == 0) t0 = now;
                if (stop || now - t0 > kWaitLimitNs) {
                    if (!stop) {
                        atomicExch(a.sync + 1, 1u);
                        if (a.status && atomicCAS(a.status, 0u, (uint32_t)WAIT_PEER) == 0u) a.status[1] = missing;
                    }
                    good = false;
                    break;
                }
            }
        }
        if (!good) break;
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int idx = first + b, k = idx / a.tp, r = idx - k * a.tp, e = tid + k * kThreads;
            if (idx < packets && e < a.hidden) {
                sum = r == 0 ? __uint_as_float(v[b].x) : __fadd_rn(sum, __uint_as_float(v[b].x));  // rank order; 0 + y0 = y0
                if (r == a.tp - 1) out[e] = bf16_rne(__fadd_rn(in[e], bf16_rne(sum)));
            }
        }
    }
    if (tid == 0) *ok_smem = 1;
    __syncthreads();
    if (!good) *ok_smem = 0;
    __syncthreads();
    return *ok_smem != 0;
}

// The same exchange in two stages, for many ranks: read directly, every CTA fetches hidden x tp packets from L2 (256 KiB
// at 8 ranks, 38 MB per exchange over the GPU).  Here a CTA sums only its slice of the row (one thread per element, the
// element's tp packets requested together), writes the result to `reduced`, the GPU's CTAs meet at a grid-wide barrier and
// everyone reads the finished row: one more barrier, an eighth of the reads.
__device__ __forceinline__ bool gather_exchange_sliced(const StepDev &a, uint32_t exchange, uint32_t tag, const float *in, float *out,
                                                       uint32_t barrier, uint32_t *ok_smem, int tid) {
    const uint2 *base = a.ll[a.rank] + (size_t)(exchange & 1u) * a.tp * a.hidden;
    int e0, e1;
    cta_rows(a.hidden, e0, e1);
    bool good = true;
    for (int e = e0 + tid; e < e1; e += kThreads) {
        uint2 v[kTpMaxRanks];
        uint32_t missing = (1u << a.tp) - 1u;
        unsigned long long t0 = 0;
        for (uint32_t spin = 1; missing; ++spin) {
#pragma unroll
            for (int r = 0; r < kTpMaxRanks; ++r)
                if (missing >> r & 1u)
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];"
                                 : "=r"(v[r].x), "=r"(v[r].y)
                                 : "l"(base + (size_t)r * a.hidden + e)
                                 : "memory");
#pragma unroll
            for (int r = 0; r < kTpMaxRanks; ++r)
                if ((missing >> r & 1u) && v[r].y == tag) missing &= ~(1u << r);
            if (missing && (spin & 63u) == 0) {
                uint32_t stop;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(stop) : "l"(a.sync + 1) : "memory");
                const unsigned long long now = global_ns();
                if (t0 == 0) t0 = now;
                if (stop || now - t0 > kWaitLimitNs) {
                    if (!stop) {
                        atomicExch(a.sync + 1, 1u);
                        if (a.status && atomicCAS(a.status, 0u, (uint32_t)WAIT_PEER) == 0u) a.status[1] = missing;
                    }
                    good = false;
                    break;
                }
            }
        }
        if (!good) break;
        float sum = __uint_as_float(v[0].x);  // rank order; 0 + y0 = y0
#pragma unroll
        for (int r = 1; r < kTpMaxRanks; ++r)
            if (r < a.tp) sum = __fadd_rn(sum, __uint_as_float(v[r].x));
        a.reduced[e] = bf16_rne(__fadd_rn(in[e], bf16_rne(sum)));
    }
    if (__syncthreads_or(!good)) return false;  // the abort word is up: the other CTAs leave at the barrier
    if (!grid_barrier(a, barrier, ok_smem, [](int, int) {})) return false;
    for (int j = tid * 4; j < a.hidden; j += kThreads * 4)
        *reinterpret_cast<float4 *>(out + j) = __ldcg(reinterpret_cast<const float4 *>(a.reduced + j));
    __syncthreads();
    return true;
}

// norm_quantize of a row that is already in shared memory
template <class T>
__device__ __forceinline__ float prologue_rmsnorm_shared(const float *x, const typename T::storage *gain, float eps, int K, int8_t *sq,
                                                         float *row, PrologueShared &ps, int tid) {
    for (int j = tid * 4; j < K; j += kThreads * 4) *reinterpret_cast<float4 *>(row + j) = *reinterpret_cast<const float4 *>(x + j);
    __syncthreads();
    return rmsnorm_row<T>(gain, eps, K, sq, row, ps, tid);
}


template <class T, bool TRACE>
__global__ void __launch_bounds__(kThreads, 1) decode_layers_tp_kernel(const StepDev a) {
    typedef typename T::storage S;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    StepSharedTp &tp = *reinterpret_cast<StepSharedTp *>(smem_raw);
    StepSharedOf<false> &sh = tp.base;
    const int tid = threadIdx.x;
    const uint32_t pos = a.control[1];
    if (pos >= (uint32_t)a.capacity) {  // every CTA of every rank takes this branch: nobody waits for anybody
        if (blockIdx.x == 0 && tid == 0 && a.status && atomicCAS(a.status, 0u, (uint32_t)FAULT_CACHE_RANGE) == 0u) a.status[1] = pos;
        return;
    }
    const int end = (int)pos + 1;
    const int q_width = a.q_heads * kHeadDim, qkv_width = (a.q_heads + 2 * a.kv_heads) * kHeadDim;  // this rank's share
    const uint32_t tag0 = *reinterpret_cast<const volatile uint32_t *>(a.seq) + 1u;  // tag of this step's first exchange
    for (int j = tid; j < a.hidden; j += kThreads) tp.hidden[j] = load_one_cg<T>(static_cast<const S *>(a.hidden_io) + j);
    __syncthreads();
    // the layer's barriers in step order: attention, O, (sliced exchange of O), down, (sliced exchange of down)
    const int per_layer = a.sliced ? 5 : 3;
    const int BAR_TP_ATTENTION = 1, BAR_TP_O = 2, BAR_TP_XO = 3, BAR_TP_DOWN = a.sliced ? 4 : 3, BAR_TP_XDOWN = 5;
    const auto ordinal = [per_layer](int l, int which) { return (uint32_t)(l * per_layer + which); };
    long long *trace = TRACE && a.trace && tid == 0 ? a.trace + (size_t)blockIdx.x * a.n_layers * kTracePoints : nullptr;
    for (int l = 0; l < a.n_layers; ++l) {
        const LayerDev L = a.layers[l];
        auto mark = [&](int point) {
            if (TRACE && trace) trace[l * kTracePoints + point] = clock64();
        };
        const uint32_t x_o = 2u * l, x_down = 2u * l + 1u;  // the layer's two exchanges
        mark(TP_START);
        // norm1 + quantize -> this rank's Q|K|V heads
        float s = prologue_rmsnorm_shared<T>(tp.hidden, static_cast<const S *>(L.norm1), a.eps, a.hidden, sh.codes, sh.row, sh.ps, tid);
        __syncthreads();
        mark(TP_NORM1);
        project_any<T, PRJ_PLAIN>(a, L.qkv, nullptr, L.qkv_s, nullptr, qkv_width, a.hidden, s, sh.codes, sh.red, nullptr,
                                  static_cast<S *>(a.qkv), tid);
        mark(TP_QKV);
        mark(TP_ARRIVE1);
        if (!grid_barrier(a, ordinal(l, BAR_TP_ATTENTION), &sh.ok, [&](int i, int n) {
                request_cache(a, L, end, i, n);
                request_rows(L.o, q_width, a.hidden, 0, 1ll << 40, i, n);
            }))
            return;
        mark(TP_PASS1);
        attention_phase<T>(a, L, sh.att.units, nullptr, end, tid, nullptr);
        mark(TP_ATTENTION);
        if (!grid_barrier(a, ordinal(l, BAR_TP_O), &sh.ok, [&](int i, int n) {
                request_rows(L.gate, a.hidden, a.inter, 0, a.ahead_bytes, i, n);
                request_rows(L.up, a.hidden, a.inter, 0, a.ahead_bytes, i, n);
            }))
            return;
        mark(TP_PASS2);
        // quantize(this rank's attention heads) -> partial O, sent to every rank
        s = prologue_plain<T>(static_cast<const S *>(a.attn), q_width, sh.codes, sh.row, sh.ps, tid);
        __syncthreads();
        mark(TP_QUANT_O);
        project_any<T, PRJ_PUSH>(a, L.o, nullptr, L.o_s, nullptr, a.hidden, q_width, s, sh.codes, sh.red, nullptr, nullptr, tid, x_o,
                                 tag0 + x_o);
        mark(TP_O);
        if (a.sliced ? !gather_exchange_sliced(a, x_o, tag0 + x_o, tp.hidden, tp.residual, ordinal(l, BAR_TP_XO), &sh.ok, tid)
                     : !gather_exchange(a, x_o, tag0 + x_o, tp.hidden, tp.residual, &sh.ok, tid))
            return;
        mark(TP_PASS3);
        // norm2 + quantize -> this rank's gate|up channels + SwiGLU
        s = prologue_rmsnorm_shared<T>(tp.residual, static_cast<const S *>(L.norm2), a.eps, a.hidden, sh.codes, sh.row, sh.ps, tid);
        __syncthreads();
        mark(TP_NORM2);
        project_any<T, PRJ_SWIGLU>(a, L.gate, L.up, L.gate_s, L.up_s, a.inter, a.hidden, s, sh.codes, sh.red, nullptr,
                                   static_cast<S *>(a.act), tid);
        mark(TP_GATE_UP);
        if (!grid_barrier(a, ordinal(l, BAR_TP_DOWN), &sh.ok,
                          [&](int i, int n) { request_rows(L.down, a.inter, a.hidden, 0, a.ahead_bytes, i, n); }))
            return;
        mark(TP_PASS4);
        // quantize(this rank's act channels) -> partial down, sent to every rank
        s = prologue_plain<T>(static_cast<const S *>(a.act), a.inter, sh.codes, sh.row, sh.ps, tid);
        __syncthreads();
        mark(TP_QUANT_DOWN);
        project_any<T, PRJ_PUSH>(a, L.down, nullptr, L.down_s, nullptr, a.hidden, a.inter, s, sh.codes, sh.red, nullptr, nullptr, tid,
                                 x_down, tag0 + x_down);
        mark(TP_DOWN);
        if (l + 1 < a.n_layers) request_rows(a.layers[l + 1].qkv, a.hidden, qkv_width, 0, a.ahead_bytes, tid, kThreads);
        if (a.sliced ? !gather_exchange_sliced(a, x_down, tag0 + x_down, tp.residual, tp.hidden, ordinal(l, BAR_TP_XDOWN), &sh.ok, tid)
                     : !gather_exchange(a, x_down, tag0 + x_down, tp.residual, tp.hidden, &sh.ok, tid))
            return;
        mark(TP_PASS5);
    }
    if (blockIdx.x == 0) {
        for (int j = tid; j < a.hidden; j += kThreads) T::store(static_cast<S *>(a.hidden_io) + j, tp.hidden[j]);
        // every CTA of this rank read the tag base before it sent its first packet, and this CTA has seen all packets
        if (tid == 0) a.seq[0] = tag0 - 1u + 2u * (uint32_t)a.n_layers;
    }
}

}  // namespace
}  // namespace w8a8

using namespace w8a8;

struct qwen3_decode_plan {
    uint32_t magic;
    int device, dtype, grid;
    StepDev dev;          // kernel argument; `layers` and the work buffers are device allocations owned by the plan
    void *layers_dev;
    void *work;           // residual | qkv | attention | act | scratch | {barrier words, attention counters}, one allocation
    size_t clear_bytes;   // barrier words + counters: zeroed in stream order before every step
    void *trace;          // W8A8_DECODE_TRACE=1 at creation: cycle counts of the last step (qwen3_decode_plan_trace)
};

namespace {

constexpr uint32_t kPlanMagic = 0x51334450u;  // "Q3DP"

bool valid_plan(const qwen3_decode_plan *p) { return p && p->magic == kPlanMagic; }
bool valid_matrix(const w8a8_weight *w) { return w && w->magic == kWeightMagic; }
size_t round_up(size_t n, size_t to) { return (n + to - 1) / to * to; }

int env_int(const char *name, int fallback) {
    const char *v = std::getenv(name);
    return v && *v ? std::atoi(v) : fallback;
}

}  // namespace

#define REQUIRE(cond, code)         \
    do {                            \
        if (!(cond)) return (code); \
    } while (0)

namespace w8a8 {
cudaError_t init_decode_layers() {
    const int smem = (int)sizeof(StepShared);
    cudaError_t e = cudaFuncSetAttribute(decode_layers_kernel<Bf16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_layers_kernel<F32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_layers_kernel<Bf16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_layers_kernel<F32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    const int smem_tp = (int)sizeof(StepSharedTp);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_layers_tp_kernel<Bf16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tp);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_layers_tp_kernel<F32, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tp);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_layers_tp_kernel<Bf16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tp);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_layers_tp_kernel<F32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tp);
    return e;
}
}  // namespace w8a8

extern "C" {

int qwen3_decode_plan_create(const qwen3_layer_desc *layers, int n_layers, int hidden, int q_heads, int kv_heads, int intermediate,
                             int capacity, float eps, const float *rope_table, int dtype, qwen3_decode_plan_t *plan_out) {
    REQUIRE(device_status_ptr(), W8A8_ERR_NOT_INITIALIZED);
    REQUIRE(layers && plan_out && rope_table && n_layers > 0, W8A8_ERR_BAD_ARG);
    REQUIRE(dtype == W8A8_BF16 || dtype == W8A8_F32, W8A8_ERR_BAD_ARG);
    REQUIRE(hidden > 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && intermediate > 0, W8A8_ERR_BAD_ARG);
    REQUIRE(capacity > 0 && capacity <= kUnitMaxContext, W8A8_ERR_BAD_ARG);
    const int q_width = q_heads * kHeadDim, qkv_width = (q_heads + 2 * kv_heads) * kHeadDim;
    // every row a lane slice of 16 bytes, every vector of the carrier whole, at most three rounds of 4096 bytes
    REQUIRE(hidden % 16 == 0 && intermediate % 16 == 0, W8A8_ERR_UNSUPPORTED);
    REQUIRE(hidden <= kMaxK && q_width <= kMaxK && intermediate <= kMaxK, W8A8_ERR_UNSUPPORTED);
    REQUIRE(q_heads <= kAttnSplitMaxUnits, W8A8_ERR_UNSUPPORTED);
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return fail_cuda(cudaGetLastError(), "cudaGetDevice");
    int cooperative = 0;
    cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device);
    REQUIRE(cooperative, W8A8_ERR_UNSUPPORTED);
    int per_sm = 0;
    cudaError_t e = dtype == W8A8_BF16
                        ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel<Bf16, false>, kThreads, sizeof(StepShared))
                        : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel<F32, false>, kThreads, sizeof(StepShared));
    if (e != cudaSuccess) return fail_cuda(e, "occupancy of the decode kernel");
    REQUIRE(per_sm >= 1, W8A8_ERR_UNSUPPORTED);
    int grid = sm_count();  // one CTA per SM
    const int forced = env_int("W8A8_DECODE_CTAS", 0);
    if (forced > 0 && forced < grid) grid = forced;
    // rows one CTA owns in the widest projection (row pairs count twice)
    const int widest = std::max(std::max(qkv_width, hidden), 2 * intermediate);
    REQUIRE((widest + grid - 1) / grid + 1 <= kMaxCtaRows, W8A8_ERR_UNSUPPORTED);

    std::vector<LayerDev> table((size_t)n_layers);
    for (int l = 0; l < n_layers; ++l) {
        const qwen3_layer_desc &d = layers[l];
        REQUIRE(valid_matrix(d.qkv) && valid_matrix(d.o) && valid_matrix(d.gate) && valid_matrix(d.up) && valid_matrix(d.down),
                W8A8_ERR_BAD_ARG);
        REQUIRE(d.norm1 && d.norm2 && d.q_gain && d.k_gain && d.k_cache && d.v_cache, W8A8_ERR_BAD_ARG);
        REQUIRE(d.qkv->N == qkv_width && d.qkv->K == hidden && d.o->N == hidden && d.o->K == q_width, W8A8_ERR_BAD_ARG);
        REQUIRE(d.gate->N == intermediate && d.gate->K == hidden && d.up->N == intermediate && d.up->K == hidden, W8A8_ERR_BAD_ARG);
        REQUIRE(d.down->N == hidden && d.down->K == intermediate, W8A8_ERR_BAD_ARG);
        REQUIRE((reinterpret_cast<uintptr_t>(d.norm1) & 15u) == 0 && (reinterpret_cast<uintptr_t>(d.norm2) & 15u) == 0 &&
                    (reinterpret_cast<uintptr_t>(d.k_cache) & 15u) == 0 && (reinterpret_cast<uintptr_t>(d.v_cache) & 15u) == 0,
                W8A8_ERR_ALIGNMENT);
        LayerDev &t = table[(size_t)l];
        t.norm1 = d.norm1; t.norm2 = d.norm2; t.q_gain = d.q_gain; t.k_gain = d.k_gain;
        t.qkv = d.qkv->w; t.qkv_s = d.qkv->w_scale;
        t.o = d.o->w; t.o_s = d.o->w_scale;
        t.gate = d.gate->w; t.gate_s = d.gate->w_scale;
        t.up = d.up->w; t.up_s = d.up->w_scale;
        t.down = d.down->w; t.down_s = d.down->w_scale;
        t.k_cache = d.k_cache; t.v_cache = d.v_cache;
    }

    qwen3_decode_plan *p = new (std::nothrow) qwen3_decode_plan();
    REQUIRE(p, W8A8_ERR_CUDA);
    p->device = device; p->dtype = dtype; p->grid = grid; p->trace = nullptr;
    const size_t el = dtype == W8A8_BF16 ? 2 : 4;
    // the same split count qwen3_attention launches for one row (forward_glue.cu), so that both give the same bits
    const int splits = attention_splits(q_heads);
    const size_t b_hidden = round_up((size_t)hidden * el, 256), b_qkv = round_up((size_t)qkv_width * el, 256);
    const size_t b_attn = round_up((size_t)q_width * el, 256), b_act = round_up((size_t)intermediate * el, 256);
    const size_t b_scratch = round_up((size_t)q_heads * splits * kUnitRecord * sizeof(float), 256);
    // barrier words, then the attention counters, then the published row maxima
    p->clear_bytes = round_up(16 + ((size_t)q_heads + 2 * (size_t)n_layers) * sizeof(uint32_t), 16);
    const size_t b_reduced = round_up((size_t)hidden * sizeof(float), 256);
    const size_t total = b_hidden + b_qkv + b_attn + b_act + b_scratch + b_reduced + round_up(p->clear_bytes, 256);
    e = cudaMalloc(&p->work, total);
    if (e == cudaSuccess) e = cudaMemset(p->work, 0, total);
    if (e == cudaSuccess) e = cudaMalloc(&p->layers_dev, table.size() * sizeof(LayerDev));
    if (e == cudaSuccess) e = cudaMemcpy(p->layers_dev, table.data(), table.size() * sizeof(LayerDev), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(p->work);
        cudaFree(p->layers_dev);
        delete p;
        return fail_cuda(e, "decode plan allocation");
    }
    char *at = static_cast<char *>(p->work);
    StepDev &s = p->dev;
    s.layers = static_cast<const LayerDev *>(p->layers_dev);
    s.n_layers = n_layers; s.hidden = hidden; s.q_heads = q_heads; s.kv_heads = kv_heads; s.inter = intermediate;
    s.capacity = capacity; s.splits = splits; s.eps = eps; s.rope = rope_table; s.control = nullptr; s.hidden_io = nullptr;
    s.residual = at; at += b_hidden;
    s.qkv = at; at += b_qkv;
    s.attn = at; at += b_attn;
    s.act = at; at += b_act;
    s.scratch = reinterpret_cast<float *>(at); at += b_scratch;
    s.reduced = reinterpret_cast<float *>(at); at += b_reduced;
    s.sync = reinterpret_cast<uint32_t *>(at);
    s.counters = s.sync + 4;
    s.maxima = s.counters + q_heads;
    s.status = device_status_ptr();
    s.seq = nullptr; s.rank = 0; s.tp = 0; s.sliced = 0;
    for (int r = 0; r < kTpMaxRanks; ++r) s.ll[r] = nullptr;
    s.trace = nullptr;
    if (env_int("W8A8_DECODE_TRACE", 0)) {
        const size_t words = (size_t)grid * n_layers * kTracePoints;
        if (cudaMalloc(&p->trace, words * sizeof(long long)) == cudaSuccess) {
            cudaMemset(p->trace, 0, words * sizeof(long long));
            s.trace = static_cast<long long *>(p->trace);
        } else {
            p->trace = nullptr;
            (void)cudaGetLastError();
        }
    }
    s.ahead_bytes = (long long)env_int("W8A8_DECODE_AHEAD_KB", 64) * 1024;
    s.ahead_more = (long long)env_int("W8A8_DECODE_AHEAD_MORE_KB", 0) * 1024;
    s.ahead_rows = env_int("W8A8_DECODE_AHEAD_BATCHES", 1);
    p->magic = kPlanMagic;
    *plan_out = p;
    return W8A8_OK;
}

int qwen3_decode_plan_destroy(qwen3_decode_plan_t plan) {
    if (!plan) return W8A8_OK;
    REQUIRE(valid_plan(plan), W8A8_ERR_BAD_ARG);
    plan->magic = 0;
    cudaFree(plan->work);
    cudaFree(plan->layers_dev);
    cudaFree(plan->trace);
    delete plan;
    return W8A8_OK;
}

int qwen3_decode_plan_set_peers(qwen3_decode_plan_t plan, void *const *packet_buffers, uint32_t *seq, int rank, int tp) {
    REQUIRE(valid_plan(plan) && packet_buffers && seq, W8A8_ERR_BAD_ARG);
    REQUIRE(tp >= 1 && tp <= kTpMaxRanks && rank >= 0 && rank < tp, W8A8_ERR_BAD_ARG);
    for (int r = 0; r < tp; ++r) REQUIRE(packet_buffers[r] && (reinterpret_cast<uintptr_t>(packet_buffers[r]) & 7u) == 0, W8A8_ERR_BAD_ARG);
    StepDev &s = plan->dev;
    for (int r = 0; r < kTpMaxRanks; ++r) s.ll[r] = r < tp ? static_cast<uint2 *>(packet_buffers[r]) : nullptr;
    s.seq = seq; s.rank = rank; s.tp = tp;
    // from four ranks on a CTA sums only its slice of an exchanged row (gather_exchange_sliced); W8A8_DECODE_SLICED=0/1 forces either
    s.sliced = env_int("W8A8_DECODE_SLICED", tp >= 4 ? 1 : 0) != 0;
    return W8A8_OK;
}

int qwen3_decode_plan_trace(qwen3_decode_plan_t plan, int64_t *cycles, size_t capacity, int *ctas, int *layers, int *points) {
    REQUIRE(valid_plan(plan) && ctas && layers && points, W8A8_ERR_BAD_ARG);
    *ctas = plan->grid;
    *layers = plan->dev.n_layers;
    *points = kTracePoints;
    REQUIRE(plan->trace, W8A8_ERR_UNSUPPORTED);
    const size_t words = (size_t)plan->grid * plan->dev.n_layers * kTracePoints;
    if (!cycles) return W8A8_OK;
    REQUIRE(capacity >= words, W8A8_ERR_BAD_ARG);
    cudaError_t e = cudaMemcpy(cycles, plan->trace, words * sizeof(long long), cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? W8A8_OK : fail_cuda(e, "decode trace read-back");
}

int qwen3_decode_layers(qwen3_decode_plan_t plan, void *hidden, const uint32_t *control, void *stream) {
    REQUIRE(valid_plan(plan) && hidden && control, W8A8_ERR_BAD_ARG);
    REQUIRE((reinterpret_cast<uintptr_t>(hidden) & 15u) == 0, W8A8_ERR_ALIGNMENT);
    cudaStream_t s = (cudaStream_t)stream;
    StepDev args = plan->dev;
    args.hidden_io = hidden;
    args.control = control;
    cudaError_t e = cudaMemsetAsync(args.sync, 0, plan->clear_bytes, s);
    if (e != cudaSuccess) return fail_cuda(e, "decode barrier reset");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)plan->grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = sizeof(StepShared);
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const bool bf16 = plan->dtype == W8A8_BF16;
    if (plan->dev.tp > 0) {
        cfg.dynamicSmemBytes = sizeof(StepSharedTp);
        if (plan->trace)
            e = bf16 ? cudaLaunchKernelEx(&cfg, decode_layers_tp_kernel<Bf16, true>, args)
                     : cudaLaunchKernelEx(&cfg, decode_layers_tp_kernel<F32, true>, args);
        else
            e = bf16 ? cudaLaunchKernelEx(&cfg, decode_layers_tp_kernel<Bf16, false>, args)
                     : cudaLaunchKernelEx(&cfg, decode_layers_tp_kernel<F32, false>, args);
    } else if (plan->trace)
        e = bf16 ? cudaLaunchKernelEx(&cfg, decode_layers_kernel<Bf16, true>, args) : cudaLaunchKernelEx(&cfg, decode_layers_kernel<F32, true>, args);
    else
        e = bf16 ? cudaLaunchKernelEx(&cfg, decode_layers_kernel<Bf16, false>, args) : cudaLaunchKernelEx(&cfg, decode_layers_kernel<F32, false>, args);
    return e == cudaSuccess ? W8A8_OK : fail_cuda(e, "decode step launch");
}

}  // extern "C"
