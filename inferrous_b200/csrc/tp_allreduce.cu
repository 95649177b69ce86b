// One-shot all-reduce of the row-split projections' partial outputs over peer memory (NVLink / NVSwitch).
//
// No counterpart in the reference (it is single-GPU: `CudaContext::new(0)`, crates/inferrous-qwen3/src/gpu.rs:248).
// Under tensor parallelism the O and down projections leave one partial [M,4096] per rank; in decode that is
// 8-128 KiB, far below the size where a ring or tree pays for its latency.  One kernel per rank does:
//   push    every CTA copies its slice of the local partial into slot[rank] of EVERY rank's staging buffer
//           with plain 16-byte peer stores, fences at system scope and bumps a per-source arrival counter in
//           each destination's flag pad (red.release.sys);
//   wait    it then polls its OWN flag pad until every source has delivered all its slices (bounded: about two
//           seconds, then an error code in the status word and a clean exit);
//   reduce  it sums its slice over the tp slots in rank order in fp32 and writes bf16(sum): the result is the
//           same on every rank and does not depend on timing.
// Counters only ever grow (one arrival per source rank and call), and the staging buffer has two halves used alternately, so nothing is
// reset between calls and a fast rank cannot overwrite data a slow rank still reads.  The call number lives in
// device memory and is advanced by the kernel itself, which keeps a captured graph replayable.
// Only plain loads and stores touch peer memory: no TMA, no multicast objects.
#include "common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace w8a8 {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kThreads = 256;
constexpr int kMaxCtas = 64;  // all CTAs of a call must be co-resident: they wait for each other's pushes

struct TpDev {
    const void *partial;
    void *out;
    size_t n_el;
    size_t slot_el;          // elements per slot; a buffer holds [2 halves][tp slots][slot_el]
    void *bufs[kMaxRanks];   // staging buffer of every rank (peer pointers)
    uint32_t *flags[kMaxRanks];  // flag pad of every rank: [tp] arrival counters
    uint32_t *seq;           // local: [0] call number, [1] CTAs finished, [2] CTAs that have pushed, in the current call
    int rank, tp;
    uint32_t *status;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t *p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <class T>
__global__ void __launch_bounds__(kThreads) tp_allreduce_kernel(const TpDev a) {
    typedef typename T::storage S;
    constexpr int V = T::kVec;
    __shared__ uint32_t s_call;
    __shared__ int s_ok;
    dependency_wait();
    if (threadIdx.x == 0) {
        s_call = *reinterpret_cast<volatile uint32_t *>(a.seq);  // nobody advances it before every CTA has pushed
        s_ok = 1;
    }
    __syncthreads();
    const uint32_t call = s_call;
    const size_t half = (size_t)(call & 1u) * a.tp * a.slot_el;
    const size_t nvec = a.n_el / V;
    const size_t per = (nvec + gridDim.x - 1) / gridDim.x;
    const size_t v0 = (size_t)blockIdx.x * per, v1 = min(nvec, v0 + per);

    // ---- push my slice of the local partial into slot[rank] of every rank ----
    const S *src = static_cast<const S *>(a.partial);
    for (size_t v = v0 + threadIdx.x; v < v1; v += kThreads) {
        const uint4 x = *reinterpret_cast<const uint4 *>(src + v * V);
        for (int p = 0; p < a.tp; ++p) {
            S *dst = static_cast<S *>(a.bufs[p]) + half + (size_t)a.rank * a.slot_el;
            *reinterpret_cast<uint4 *>(dst + v * V) = x;
        }
    }
    __threadfence_system();
    __syncthreads();
    // The CTA that completes this rank's push (whatever the grid size of this call) tells every rank: one
    // arrival per source rank and call, so the counters do not depend on how a call was cut into CTAs.
    __shared__ int s_last;
    if (threadIdx.x == 0) {
        const uint32_t pushed = atomicAdd(a.seq + 2, 1u) + 1u;
        s_last = pushed == gridDim.x;
        if (s_last) a.seq[2] = 0;
        __threadfence_system();
    }
    __syncthreads();
    if (s_last && threadIdx.x < a.tp) red_release_sys_add(a.flags[threadIdx.x] + a.rank, 1u);

    // ---- wait until every source rank has delivered its partial for this call ----
    const uint32_t want = call + 1u;
    if (threadIdx.x < a.tp) {
        const uint32_t *f = a.flags[a.rank] + threadIdx.x;
        unsigned long long t0 = 0;
        uint32_t spin = 0;
        while ((int32_t)(ld_acquire_sys(f) - want) < 0) {
            if ((++spin & 63u) == 0) {
                const unsigned long long now = global_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > kWaitLimitNs) {
                    if (a.status && atomicCAS(a.status, 0u, (uint32_t)WAIT_PEER) == 0u) a.status[1] = (uint32_t)threadIdx.x;
                    s_ok = 0;
                    break;
                }
            }
        }
    }
    __syncthreads();

    // ---- reduce my slice over the slots, in rank order, in fp32 ----
    if (s_ok) {
        const S *mine = static_cast<const S *>(a.bufs[a.rank]) + half;
        S *out = static_cast<S *>(a.out);
        for (size_t v = v0 + threadIdx.x; v < v1; v += kThreads) {
            float sum[V];
#pragma unroll
            for (int i = 0; i < V; ++i) sum[i] = 0.0f;
            for (int r = 0; r < a.tp; ++r) {
                const uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(mine + (size_t)r * a.slot_el + v * V));
                const S *e = reinterpret_cast<const S *>(&raw);
                float x[V];
#pragma unroll
                for (int i = 0; i < V; ++i) x[i] = T::load(e + i);
#pragma unroll
                for (int i = 0; i < V; ++i) sum[i] = __fadd_rn(sum[i], x[i]);
            }
#pragma unroll
            for (int i = 0; i < V; ++i) sum[i] = bf16_rne(sum[i]);
            Vec<T>::store(out + v * V, sum);
        }
    }

    // ---- the last CTA to finish advances the call number ----
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t done = atomicAdd(a.seq + 1, 1u) + 1u;
        if (done == gridDim.x) {
            a.seq[1] = 0;
            __threadfence();
            a.seq[0] = call + 1u;
        }
    }
}

// Consumer of the packets a row-split projection pushed with EPI_PUSH (gemv.cu): every thread waits (bounded) for the
// tp packets of its element to carry the tag of the current call, adds them in rank order in fp32, rounds to bf16 and
// optionally adds the residual -- what `linear_residual` does on one GPU, with the sum over ranks in between.  No CTA
// waits for another CTA; the last one to finish advances the call number that the next push reads.
template <class T>
__global__ void __launch_bounds__(kThreads) tp_reduce_kernel(const uint2 *__restrict__ ll, uint32_t *seq, const typename T::storage *residual,
                                                             typename T::storage *out, typename T::storage *combined, size_t n_el,
                                                             int tp, unsigned long long slot, uint32_t *status) {
    dependency_wait();
    const uint32_t call = *reinterpret_cast<volatile uint32_t *>(seq);
    const uint32_t want = call + 1u;
    const uint2 *base = ll + (size_t)(call & 1u) * tp * slot;
    for (size_t e = (size_t)blockIdx.x * kThreads + threadIdx.x; e < n_el; e += (size_t)gridDim.x * kThreads) {
        float sum = 0.0f;
        bool ok = true;
        for (int r = 0; r < tp && ok; ++r) {
            const uint2 *p = base + (size_t)r * slot + e;
            uint2 v;
            unsigned long long t0 = 0;
            uint32_t spin = 0;
            for (;;) {
                asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
                if (v.y == want) break;
                if ((++spin & 255u) == 0) {
                    const unsigned long long now = global_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > kWaitLimitNs) {
                        if (status && atomicCAS(status, 0u, (uint32_t)WAIT_PEER) == 0u) status[1] = (uint32_t)r;
                        ok = false;
                        break;
                    }
                }
            }
            sum = __fadd_rn(sum, __uint_as_float(v.x));
        }
        if (!ok) continue;
        const float y = bf16_rne(sum);
        if (out) T::store(out + e, y);
        if (combined) T::store(combined + e, bf16_rne(__fadd_rn(T::load(residual + e), y)));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t done = atomicAdd(seq + 1, 1u) + 1u;
        if (done == gridDim.x) {
            seq[1] = 0;
            __threadfence();
            seq[0] = call + 1u;
        }
    }
}

}  // namespace

cudaError_t launch_tp_reduce(const uint2 *ll, uint32_t *seq, const void *residual, void *out, void *combined, size_t n_el, int dtype,
                             int tp, unsigned long long slot, cudaStream_t s) {
    if (!ll || !seq || tp < 1 || tp > kMaxRanks || n_el == 0 || n_el > slot || (!out && !combined) || (combined && !residual))
        return cudaErrorInvalidValue;
    int grid = (int)((n_el + 4 * kThreads - 1) / (4 * kThreads));
    grid = grid < 1 ? 1 : (grid > 128 ? 128 : grid);
    if (dtype == 0)
        return launch_kernel(tp_reduce_kernel<Bf16>, dim3(grid), dim3(kThreads), (size_t)0, s, ll, seq, (const uint16_t *)residual,
                             (uint16_t *)out, (uint16_t *)combined, n_el, tp, slot, device_status_ptr());
    return launch_kernel(tp_reduce_kernel<F32>, dim3(grid), dim3(kThreads), (size_t)0, s, ll, seq, (const float *)residual, (float *)out,
                         (float *)combined, n_el, tp, slot, device_status_ptr());
}

cudaError_t launch_tp_allreduce(const void *partial, void *out, size_t n_el, int dtype, void *const *bufs, uint32_t *const *flags,
                                uint32_t *seq, int rank, int tp, size_t slot_el, cudaStream_t s) {
    if (tp < 1 || tp > kMaxRanks || rank < 0 || rank >= tp || n_el == 0 || n_el > slot_el) return cudaErrorInvalidValue;
    const int vec = dtype == 0 ? 8 : 4;
    if (n_el % vec != 0 || slot_el % vec != 0) return cudaErrorInvalidValue;
    TpDev d{};
    d.partial = partial; d.out = out; d.n_el = n_el; d.slot_el = slot_el; d.seq = seq; d.rank = rank; d.tp = tp;
    for (int p = 0; p < tp; ++p) { d.bufs[p] = bufs[p]; d.flags[p] = flags[p]; }
    d.status = device_status_ptr();
    // one CTA per 2048 vectors, at most kMaxCtas: the same function of n_el on every rank
    const size_t nvec = n_el / vec;
    int grid = (int)((nvec + 2047) / 2048);
    if (grid > kMaxCtas) grid = kMaxCtas;
    if (grid < 1) grid = 1;
    if (dtype == 0) return launch_kernel(tp_allreduce_kernel<Bf16>, dim3(grid), dim3(kThreads), (size_t)0, s, d);
    return launch_kernel(tp_allreduce_kernel<F32>, dim3(grid), dim3(kThreads), (size_t)0, s, d);
}

}  // namespace w8a8
