// Host-side launcher interface between the C ABI (capi.cu) and the kernel files.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

struct w8a8_weight {
    uint32_t magic;
    int device;
    const int8_t *w;
    const float *w_scale;
    int N, K;
    CUtensorMap map_rows256;  // [N,K] uint8, box 128 bytes x 256 rows, SWIZZLE_128B
    CUtensorMap map_rows128;  // same with a 128-row box
    CUtensorMap map_rows96;   // same with a 96-row box
    CUtensorMap map_rows64;   // same with a 64-row box
    bool has_maps;
};

namespace w8a8 {

constexpr uint32_t kWeightMagic = 0x57384138u;  // "W8A8"
constexpr int kMaxGroup = 3;

enum QuantMode { QUANT_PLAIN = 0, QUANT_WITH_MAX = 1, QUANT_RMSNORM = 2, QUANT_SWIGLU = 3 };

struct QuantArgs {
    int mode;
    int dtype;
    const void *x;      // plain / with_max / rmsnorm input; swiglu gate
    const void *x2;     // rmsnorm gamma; swiglu up
    int64_t ld;         // row stride of x (and x2 for swiglu), elements
    int M, K;           // K = quantized row width
    float eps;
    const uint32_t *maxima_in;  // with_max
    int8_t *q;
    float *scale;
    void *y_out;             // optional pre-quant bf16 row (rmsnorm y / swiglu act), row stride K
    uint32_t *maxima_reset;  // optional
};
cudaError_t launch_quantize(const QuantArgs &a, cudaStream_t s);
cudaError_t launch_swiglu(const void *gate, const void *up, int dtype, int M, int I, int64_t ld, void *act,
                          uint32_t *maxima, cudaStream_t s);
cudaError_t launch_residual(const void *a, const void *b, int dtype, size_t n, void *out, cudaStream_t s);
cudaError_t launch_rounding_probe(const float *x, int8_t *out, size_t n, cudaStream_t s);

// Where a decode GEMV takes its quantized activation row from: codes + scale written by a quantizer kernel, or the
// quantizer folded into the GEMV's own prologue (one token; every CTA quantizes the row for itself).
enum ActivationSource { SRC_CODES = 0, SRC_WITH_MAX = 1, SRC_RMSNORM = 2 };

enum Epilogue { EPI_PLAIN = 0, EPI_RESIDUAL = 1, EPI_SWIGLU = 2, EPI_ACC = 3, EPI_ARGMAX = 4, EPI_PUSH = 5 };

// EPI_PUSH (tensor parallel, row-split projections in decode): the partial output is not written locally but sent to
// every rank as 8-byte packets {float32 bits of the bf16 value, tag}; a packet is one store, so data and tag arrive
// together and the consumer (tp_reduce) needs no fence, only to see the tag of the current call.
constexpr int kTpMaxRanks = 8;
struct PushTarget {
    uint2 *ll[kTpMaxRanks];   // packet buffer of every rank: [2 halves][tp sources][slot packets]
    const uint32_t *seq;      // local: [0] = number of completed calls
    int rank, tp;
    unsigned long long slot;  // packets per (half, source)
};

struct LinearArgs {
    const int8_t *q;
    const float *a_scale;
    int M, K;
    int count;                    // matrices in the group (1 for a plain projection; 2 for gate/up)
    const int8_t *w[kMaxGroup];
    const float *ws[kMaxGroup];
    void *out[kMaxGroup];         // y per matrix (may be null for EPI_RESIDUAL / EPI_SWIGLU)
    int n[kMaxGroup];
    int epilogue;
    const void *residual;         // EPI_RESIDUAL
    void *combined;               // EPI_RESIDUAL
    void *act;                    // EPI_SWIGLU
    uint32_t *maxima;             // EPI_SWIGLU
    int32_t *acc;                 // EPI_ACC: raw accumulators [M, n[0]]
    unsigned long long *partial_best;  // EPI_ARGMAX: [row blocks][16] packed (ordered value, ~index) per token
    int dtype;
    // ActivationSource != SRC_CODES (gemv_dp4a only, M == 1): the unquantized row and what its quantizer needs
    int src;
    const void *x;               // [K] activations in `dtype`
    const void *gamma;           // SRC_RMSNORM: gain row
    float eps;                   // SRC_RMSNORM
    const uint32_t *maxima_in;   // SRC_WITH_MAX: bit pattern of max(1e-8, max|x|), published by the producer
    uint32_t *maxima_reset;      // optional: `reset_words` words set to the bits of 1e-8f by the first CTA
    int reset_words;
    int8_t *q_out;               // optional: the codes, written by the first CTA
    float *scale_out;            // optional: the scale, written by the first CTA
    PushTarget push;             // EPI_PUSH
};
cudaError_t launch_linear_naive(const LinearArgs &a, cudaStream_t s);
cudaError_t launch_gemv_dp4a(const LinearArgs &a, cudaStream_t s);   // M <= 4
cudaError_t launch_gemv_mma(const LinearArgs &a, cudaStream_t s);    // M <= 64
// tcgen05 path: one matrix, EPI_PLAIN / EPI_RESIDUAL / EPI_ACC
cudaError_t launch_gemm_tcgen05(const LinearArgs &a, const w8a8_weight *wt, cudaStream_t s);
cudaError_t init_gemm_tcgen05();
int tcgen05_tile_channels(int M, int N);  // 256, 128 or 64: output channels per tile the launcher will use
cudaError_t launch_gemm_tcgen05_pair(const LinearArgs &a, const w8a8_weight *wt, cudaStream_t s);  // CTA pairs
cudaError_t init_gemm_tcgen05_pair();
int pair_tile_channels(int M, int N);  // 256 or 192: output channels per tile the CTA-pair launcher will use
cudaError_t make_weight_maps(w8a8_weight *wt);  // TMA descriptors of the [N,K] matrix
// [rows,K] int8 row-major -> tiled map with a box of 128 bytes of K x box_rows rows, 128-byte swizzle, zero fill.
cudaError_t encode_tile_map(CUtensorMap *map, const void *base, int rows, int K, int box_rows);
// 9..128 tokens, small and mid-sized matrices: K split over a thread-block cluster, partial sums through distributed shared memory
cudaError_t launch_gemm_cluster(const LinearArgs &a, const w8a8_weight *wt, cudaStream_t s);
cudaError_t init_gemm_cluster();
constexpr int kClusterMaxTokens = 256;
// few-token tensor-core path (weights on the MMA's M side, stream-K over output tiles x K blocks)
cudaError_t launch_gemm_skinny(const LinearArgs &a, const w8a8_weight *wt, cudaStream_t s);
cudaError_t init_gemm_skinny();
// Per-device scratch of the stream-K fix-up: int32 partial tiles and arrival counters (all zero between launches).
int32_t *skinny_scratch();
uint32_t *skinny_counters();
constexpr int kSkinnyMaxTokens = 256;
constexpr int kNoAllocMaxTokens = 16;
// Allocation-free projection: stream-K scratch in a fixed device array of the library (gemm_skinny.cu).
cudaError_t launch_linear_no_alloc(const int8_t *q, const float *a_scale, const int8_t *w, const float *w_scale, int M, int N,
                                   int K, void *y, int dtype, cudaStream_t s);
// Status words of that entry point (an expired wait), read and cleared; *present = it has run on the current device.
cudaError_t read_no_alloc_status(cudaStream_t s, uint32_t out[2], bool *present);
constexpr size_t kSkinnySlotInts = 4 * (size_t)kSkinnyMaxTokens * 32;  // one 128-channel tile: [quarter][token][32]
cudaError_t init_gemv();
cudaError_t init_quantize();
cudaError_t init_forward_glue();
cudaError_t init_batched_decode();
cudaError_t init_head_bf16();
cudaError_t init_decode_layers();

// Device status word (bounded waits report here instead of trapping).
uint32_t *device_status_ptr();  // device address of the 2-word status block of the current device
cudaError_t read_device_status(cudaStream_t s, uint32_t out[2]);

// greedy token selection fused into the head projection (gemv.cu): finish = reduce the per-block candidates
cudaError_t launch_argmax_finish(const unsigned long long *partial, int blocks, int M, uint32_t *token, float *value, cudaStream_t s);
unsigned long long *argmax_scratch();  // per device: kArgmaxMaxBlocks x 16 candidates
constexpr int kArgmaxMaxBlocks = 16384;  // head matrices up to 262144 output channels

// consumer of EPI_PUSH packets: sum over the ranks in rank order, optional residual (tp_allreduce.cu)
cudaError_t launch_tp_reduce(const uint2 *ll, uint32_t *seq, const void *residual, void *out, void *combined, size_t n_el, int dtype,
                             int tp, unsigned long long slot, cudaStream_t s);
// one-shot all-reduce over peer memory (tp_allreduce.cu)
cudaError_t launch_tp_allreduce(const void *partial, void *out, size_t n_el, int dtype, void *const *bufs, uint32_t *const *flags,
                                uint32_t *seq, int rank, int tp, size_t slot_el, cudaStream_t s);

// split-key attention (forward_glue.cu): per (row, head, split) partial results and per (row, head) arrival
// counters (zero between launches), allocated once per device
constexpr int kAttnSplitMaxUnits = 256;
constexpr int kAttnMaxSplits = 16;
constexpr size_t kAttnScratchFloats = (size_t)kAttnSplitMaxUnits * kAttnMaxSplits * 132;
float *attention_scratch();
uint32_t *attention_counters();
// Key splits launched for `units` (row, head) pairs: as many as keep units * splits within two CTAs per SM.  The resident
// decode kernel uses the same number, so that both give the same bits.
int attention_splits(int units);

// L2 prefetch hint for immutable weights (w8a8_prefetch_hint): consumed by the next launch that carries prefetch CTAs.
constexpr int kMaxPrefetchRanges = 4;
constexpr int kPrefetchMaxRows = 16;  // quantizer launches with more rows leave pending hints alone
struct PrefetchHint {
    const char *ptr[kMaxPrefetchRanges];
    unsigned long long bytes[kMaxPrefetchRanges];
    int count;
};
PrefetchHint take_prefetch_hint();

#ifdef __CUDACC__
// The whole 128-byte lines inside [base, base + bytes), dealt round-robin to the threads of `ctas` CTAs (partial
// lines at either end are left alone, so no address outside the range is ever named).
__device__ __forceinline__ void prefetch_lines(const char *base, unsigned long long bytes, int cta, int ctas) {
    const unsigned long long begin = (reinterpret_cast<unsigned long long>(base) + 127ull) & ~127ull;
    const unsigned long long end = (reinterpret_cast<unsigned long long>(base) + bytes) & ~127ull;
    if (end <= begin) return;
    const unsigned long long lines = (end - begin) / 128;
    for (unsigned long long i = (unsigned long long)cta * blockDim.x + threadIdx.x; i < lines; i += (unsigned long long)ctas * blockDim.x)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(begin + i * 128));
}

// The role of a prefetch CTA: hint every pending range, `cta` of `ctas`.
__device__ __forceinline__ void prefetch_ranges(const PrefetchHint &hint, int cta, int ctas) {
    for (int r = 0; r < hint.count; ++r) prefetch_lines(hint.ptr[r], hint.bytes[r], cta, ctas);
}
#endif

int sm_count();
// Records the failing CUDA call's text for w8a8_last_cuda_error() and returns W8A8_ERR_CUDA.
int fail_cuda(cudaError_t e, const char *what);

// Programmatic dependent launch (the reference's CLEAN_PDL switch, src/gpu.rs:317; src/graph.rs:63-127):
// when enabled, every hot-path kernel is launched with the programmatic-stream-serialization attribute,
// so it may start while its predecessor drains; each kernel's griddepcontrol.wait keeps the data order.
bool programmatic_launch_enabled();

template <class Kernel, class... Args>
cudaError_t launch_kernel(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    if (programmatic_launch_enabled()) {
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace w8a8
