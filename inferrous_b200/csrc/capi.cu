// The C ABI (include/w8a8.h): argument validation, regime selection, status reporting.
//
// Regime selection mirrors GpuModel::linear_quantized (crates/inferrous-qwen3/src/gpu.rs:450-509),
// which switches kernels on the token count: 1 -> linear, 2..31 -> linear_splitk,
// 32..255 -> linear_tiled, >= 256 (and N >= 4096) -> linear_large.  Here:
//   gemv_dp4a      weight streaming with 16-byte loads + dp4a (1 token; fused gate/up up to 4)
//   gemv_mma       weight streaming + warp-level int8 MMA (2..64 tokens, small and mid matrices)
//   gemm_skinny    TMA + tcgen05.mma kind::i8, weights on the MMA's M side, stream-K (large matrices, <= 256 tokens)
//   gemm_cluster   the same operand roles, K split over a thread-block cluster, partial sums reduced through distributed
//                  shared memory (16-50 MB matrices, 17..128 tokens)
//   gemm_tcgen05   TMA + tcgen05.mma kind::i8, 128x256 tiles, persistent (65..128 tokens)
//   gemm_tcgen05_pair  the same over CTA pairs (cta_group::2), 256x256 tiles (prefill, >= 129 tokens)
// see pick_variant() for the thresholds.
#include "../../include/w8a8.h"
#include "internal.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace w8a8 {

namespace {
constexpr int kMaxDevices = 64;
struct DeviceState {
    bool ready = false;
    int sms = 0;
    uint32_t *status = nullptr;  // 2 words: [0] wait code, [1] detail
    int32_t *sk_scratch = nullptr;   // stream-K partial tiles, zero between launches
    uint32_t *sk_counters = nullptr; // stream-K arrival counters, zero between launches
    unsigned long long *argmax = nullptr;  // per-block candidates of the fused head projection
    float *attn_scratch = nullptr;         // split-key attention: partial results
    uint32_t *attn_counters = nullptr;     // split-key attention: arrival counters, zero between launches
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;
bool g_pdl = false;
thread_local char g_err[256] = "";
thread_local PrefetchHint g_hint = {};

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int current_ready_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return g_dev[dev].ready ? dev : -1;
}
}  // namespace

bool programmatic_launch_enabled() { return g_pdl; }

PrefetchHint take_prefetch_hint() {
    const PrefetchHint h = g_hint;
    g_hint = PrefetchHint{};
    return h;
}

int fail_cuda(cudaError_t e, const char *what) {
    snprintf(g_err, sizeof g_err, "%s: %s", what, cudaGetErrorString(e));
    return W8A8_ERR_CUDA;
}

int sm_count() {
    int dev = current_ready_device();
    return dev < 0 ? 148 : g_dev[dev].sms;
}
uint32_t *device_status_ptr() {
    int dev = current_ready_device();
    return dev < 0 ? nullptr : g_dev[dev].status;
}
int32_t *skinny_scratch() {
    int dev = current_ready_device();
    return dev < 0 ? nullptr : g_dev[dev].sk_scratch;
}
unsigned long long *argmax_scratch() {
    int dev = current_ready_device();
    return dev < 0 ? nullptr : g_dev[dev].argmax;
}
int attention_splits(int units) { return std::max(1, std::min(kAttnMaxSplits, (2 * sm_count()) / std::max(1, units))); }

float *attention_scratch() {
    int dev = current_ready_device();
    return dev < 0 ? nullptr : g_dev[dev].attn_scratch;
}
uint32_t *attention_counters() {
    int dev = current_ready_device();
    return dev < 0 ? nullptr : g_dev[dev].attn_counters;
}
uint32_t *skinny_counters() {
    int dev = current_ready_device();
    return dev < 0 ? nullptr : g_dev[dev].sk_counters;
}
// After an abandoned launch (a bounded wait ran out) the scratch that every launch is meant to leave at zero may hold
// partial sums or arrival counts: return it to zero, in stream order, so that later launches are right again.
void reset_shared_scratch(cudaStream_t s) {
    int dev = current_ready_device();
    if (dev < 0) return;
    DeviceState &d = g_dev[dev];
    cudaMemsetAsync(d.sk_scratch, 0, (size_t)d.sms * kSkinnySlotInts * sizeof(int32_t), s);
    cudaMemsetAsync(d.sk_counters, 0, (size_t)d.sms * 4 * sizeof(uint32_t), s);
    cudaMemsetAsync(d.attn_counters, 0, 2 * kAttnSplitMaxUnits * sizeof(uint32_t), s);
    cudaStreamSynchronize(s);
}

cudaError_t read_device_status(cudaStream_t s, uint32_t out[2]) {
    uint32_t *p = device_status_ptr();
    if (!p) return cudaErrorInitializationError;
    cudaError_t e = cudaMemcpyAsync(out, p, 8, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(p, 0, 8, s)) != cudaSuccess) return e;
    return cudaStreamSynchronize(s);
}

}  // namespace w8a8

using namespace w8a8;

#define REQUIRE(cond, code) \
    do {                    \
        if (!(cond)) return (code); \
    } while (0)
#define CUDA_OK(expr, what)                              \
    do {                                                 \
        cudaError_t e__ = (expr);                        \
        if (e__ != cudaSuccess) return fail_cuda(e__, what); \
    } while (0)

extern "C" {

const char *w8a8_version(void) { return "0.1.0"; }

const char *w8a8_status_string(int status) {
    switch (status) {
        case W8A8_OK: return "ok";
        case W8A8_ERR_BAD_ARG: return "bad argument";
        case W8A8_ERR_ALIGNMENT: return "alignment: K must be a multiple of 128 and pointers 16-byte aligned";
        case W8A8_ERR_UNSUPPORTED: return "shape not supported by the requested kernel variant";
        case W8A8_ERR_CUDA: return "CUDA call failed";
        case W8A8_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
        case W8A8_ERR_NOT_INITIALIZED: return "w8a8_init() has not run for the current device";
        default: return "unknown status";
    }
}

const char *w8a8_last_cuda_error(void) { return g_err; }

size_t w8a8_workspace_bytes(int max_rows, int hidden, int q_width, int intermediate, size_t *offsets) {
    if (max_rows <= 0 || hidden <= 0 || q_width <= 0 || intermediate <= 0) return 0;
    const size_t rows = (size_t)max_rows;
    const size_t region[5] = {rows * (size_t)hidden, rows * (size_t)q_width, rows * (size_t)intermediate, rows * sizeof(float),
                              rows * sizeof(uint32_t)};
    size_t at = 0;
    for (int i = 0; i < 5; ++i) {
        if (offsets) offsets[i] = at;
        at += (region[i] + 255) / 256 * 256;
    }
    return at;
}

int w8a8_prefetch_hint(const void *weights, size_t bytes) {
    REQUIRE((weights != nullptr) == (bytes != 0), W8A8_ERR_BAD_ARG);
    if (!weights) {
        g_hint = PrefetchHint{};
        return W8A8_OK;
    }
    REQUIRE(g_hint.count < kMaxPrefetchRanges, W8A8_ERR_UNSUPPORTED);
    g_hint.ptr[g_hint.count] = static_cast<const char *>(weights);
    g_hint.bytes[g_hint.count] = bytes;
    ++g_hint.count;
    return W8A8_OK;
}

int w8a8_set_programmatic_launch(int enabled) {
    g_pdl = enabled != 0;
    return W8A8_OK;
}

int w8a8_init(int device) {
    REQUIRE(device >= 0 && device < kMaxDevices, W8A8_ERR_BAD_ARG);
    std::lock_guard<std::mutex> lock(g_mu);
    CUDA_OK(cudaSetDevice(device), "cudaSetDevice");
    DeviceState &d = g_dev[device];
    if (d.ready) return W8A8_OK;
    cudaDeviceProp prop;
    CUDA_OK(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    if (prop.major != 10) {
        snprintf(g_err, sizeof g_err, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return W8A8_ERR_CUDA;
    }
    d.sms = prop.multiProcessorCount;
    if (const char *e = getenv("W8A8_PDL")) g_pdl = atoi(e) != 0;
    CUDA_OK(cudaMalloc(&d.status, 8), "cudaMalloc(status)");
    CUDA_OK(cudaMemset(d.status, 0, 8), "cudaMemset(status)");
    // Scratch of the stream-K fix-up (gemm_skinny.cu): allocated once here, never in a launch call.
    const size_t sk_bytes = (size_t)d.sms * kSkinnySlotInts * sizeof(int32_t);
    CUDA_OK(cudaMalloc(&d.sk_scratch, sk_bytes), "cudaMalloc(stream-K scratch)");
    CUDA_OK(cudaMemset(d.sk_scratch, 0, sk_bytes), "cudaMemset(stream-K scratch)");
    CUDA_OK(cudaMalloc(&d.sk_counters, (size_t)d.sms * 4 * sizeof(uint32_t)), "cudaMalloc(stream-K counters)");
    CUDA_OK(cudaMemset(d.sk_counters, 0, (size_t)d.sms * 4 * sizeof(uint32_t)), "cudaMemset(stream-K counters)");
    CUDA_OK(cudaMalloc(&d.argmax, (size_t)kArgmaxMaxBlocks * 16 * sizeof(unsigned long long)), "cudaMalloc(argmax candidates)");
    CUDA_OK(cudaMalloc(&d.attn_scratch, kAttnScratchFloats * sizeof(float)), "cudaMalloc(attention scratch)");
    // arrival counters: one per (row, head) for the key splits, then one per row for the folded quantizer
    CUDA_OK(cudaMalloc(&d.attn_counters, 2 * kAttnSplitMaxUnits * sizeof(uint32_t)), "cudaMalloc(attention counters)");
    CUDA_OK(cudaMemset(d.attn_counters, 0, 2 * kAttnSplitMaxUnits * sizeof(uint32_t)), "cudaMemset(attention counters)");
    CUDA_OK(init_quantize(), "init_quantize");
    CUDA_OK(init_gemv(), "init_gemv");
    CUDA_OK(init_gemm_tcgen05(), "init_gemm_tcgen05");
    CUDA_OK(init_gemm_tcgen05_pair(), "init_gemm_tcgen05_pair");
    CUDA_OK(init_gemm_skinny(), "init_gemm_skinny");
    CUDA_OK(init_gemm_cluster(), "init_gemm_cluster");
    CUDA_OK(init_forward_glue(), "init_forward_glue");
    CUDA_OK(init_batched_decode(), "init_batched_decode");
    CUDA_OK(init_head_bf16(), "init_head_bf16");
    CUDA_OK(init_decode_layers(), "init_decode_layers");
    d.ready = true;
    return W8A8_OK;
}

int w8a8_device_status(void *stream, uint32_t *detail) {
    // Two places record an expired wait: the status word w8a8_init() allocated, and the one inside the fixed array of
    // w8a8_linear_no_alloc (which may be the only one: that entry point needs no w8a8_init).
    uint32_t fixed[2] = {0, 0};
    bool fixed_present = false;
    CUDA_OK(read_no_alloc_status((cudaStream_t)stream, fixed, &fixed_present), "read_no_alloc_status");
    const bool ready = current_ready_device() >= 0;
    REQUIRE(ready || fixed_present, W8A8_ERR_NOT_INITIALIZED);
    uint32_t words[2] = {0, 0};
    if (ready) {
        CUDA_OK(read_device_status((cudaStream_t)stream, words), "read_device_status");
        if (words[0]) reset_shared_scratch((cudaStream_t)stream);
    }
    if (!words[0]) {
        words[0] = fixed[0];
        words[1] = fixed[1];
    }
    if (detail) *detail = words[0] ? ((words[0] << 24) | (words[1] & 0xffffffu)) : 0;
    return words[0] ? W8A8_ERR_DEVICE_TIMEOUT : W8A8_OK;
}

// ---- weights ---------------------------------------------------------------------------

int w8a8_weight_create(const int8_t *w, const float *w_scale, int N, int K, w8a8_weight_t *out) {
    REQUIRE(w && w_scale && out && N > 0 && K > 0, W8A8_ERR_BAD_ARG);
    REQUIRE(K % 128 == 0 && (reinterpret_cast<uintptr_t>(w) & 127u) == 0 && aligned16(w_scale), W8A8_ERR_ALIGNMENT);
    int dev = current_ready_device();
    REQUIRE(dev >= 0, W8A8_ERR_NOT_INITIALIZED);
    w8a8_weight *wt = new (std::nothrow) w8a8_weight();
    REQUIRE(wt, W8A8_ERR_BAD_ARG);
    wt->magic = kWeightMagic;
    wt->device = dev;
    wt->w = w;
    wt->w_scale = w_scale;
    wt->N = N;
    wt->K = K;
    wt->has_maps = false;
    cudaError_t e = make_weight_maps(wt);
    if (e != cudaSuccess) {
        delete wt;
        return fail_cuda(e, "cuTensorMapEncodeTiled(weight)");
    }
    *out = wt;
    return W8A8_OK;
}

int w8a8_weight_destroy(w8a8_weight_t weight) {
    REQUIRE(weight && weight->magic == kWeightMagic, W8A8_ERR_BAD_ARG);
    weight->magic = 0;
    delete weight;
    return W8A8_OK;
}

int w8a8_weight_shape(w8a8_weight_t weight, int *N, int *K) {
    REQUIRE(weight && weight->magic == kWeightMagic, W8A8_ERR_BAD_ARG);
    if (N) *N = weight->N;
    if (K) *K = weight->K;
    return W8A8_OK;
}

// ---- quantizers ------------------------------------------------------------------------

static int check_dtype(int dtype) { return dtype == W8A8_BF16 || dtype == W8A8_F32; }
static int elem_vec(int dtype) { return dtype == W8A8_BF16 ? 8 : 4; }

static int quant_common(QuantArgs &a, void *stream) {
    REQUIRE(check_dtype(a.dtype), W8A8_ERR_BAD_ARG);
    REQUIRE(a.x && a.q && a.scale && a.M > 0 && a.K > 0 && a.ld >= a.K, W8A8_ERR_BAD_ARG);
    REQUIRE(a.K % 128 == 0 && a.ld % elem_vec(a.dtype) == 0, W8A8_ERR_ALIGNMENT);
    REQUIRE(aligned16(a.x) && aligned16(a.q) && (reinterpret_cast<uintptr_t>(a.scale) & 3u) == 0, W8A8_ERR_ALIGNMENT);
    REQUIRE(a.x2 == nullptr || aligned16(a.x2), W8A8_ERR_ALIGNMENT);
    REQUIRE(a.y_out == nullptr || aligned16(a.y_out), W8A8_ERR_ALIGNMENT);
    REQUIRE(a.K <= 24576, W8A8_ERR_UNSUPPORTED);
    REQUIRE(current_ready_device() >= 0, W8A8_ERR_NOT_INITIALIZED);
    CUDA_OK(launch_quantize(a, (cudaStream_t)stream), "launch_quantize");
    return W8A8_OK;
}

int w8a8_quantize(const void *x, int dtype, int M, int K, int64_t ldx, int8_t *q, float *scale, void *stream) {
    QuantArgs a{};
    a.mode = QUANT_PLAIN; a.dtype = dtype; a.x = x; a.ld = ldx; a.M = M; a.K = K; a.q = q; a.scale = scale;
    return quant_common(a, stream);
}

int w8a8_quantize_with_max(const void *x, int dtype, const uint32_t *maxima, int M, int K, int64_t ldx, int8_t *q,
                           float *scale, void *stream) {
    REQUIRE(maxima, W8A8_ERR_BAD_ARG);
    QuantArgs a{};
    a.mode = QUANT_WITH_MAX; a.dtype = dtype; a.x = x; a.ld = ldx; a.M = M; a.K = K; a.q = q; a.scale = scale;
    a.maxima_in = maxima;
    return quant_common(a, stream);
}

int w8a8_rmsnorm_quantize(const void *x, const void *gamma, int dtype, float eps, int M, int K, int64_t ldx, int8_t *q,
                          float *scale, void *y_out, uint32_t *maxima_reset, void *stream) {
    REQUIRE(gamma, W8A8_ERR_BAD_ARG);
    QuantArgs a{};
    a.mode = QUANT_RMSNORM; a.dtype = dtype; a.x = x; a.x2 = gamma; a.ld = ldx; a.M = M; a.K = K; a.eps = eps;
    a.q = q; a.scale = scale; a.y_out = y_out; a.maxima_reset = maxima_reset;
    return quant_common(a, stream);
}

int w8a8_swiglu_quantize(const void *gate, const void *up, int dtype, int M, int I, int64_t ld, int8_t *q, float *scale,
                         void *act_out, void *stream) {
    REQUIRE(up, W8A8_ERR_BAD_ARG);
    QuantArgs a{};
    a.mode = QUANT_SWIGLU; a.dtype = dtype; a.x = gate; a.x2 = up; a.ld = ld; a.M = M; a.K = I;
    a.q = q; a.scale = scale; a.y_out = act_out;
    return quant_common(a, stream);
}

int w8a8_swiglu(const void *gate, const void *up, int dtype, int M, int I, int64_t ld, void *act, uint32_t *maxima,
                void *stream) {
    REQUIRE(check_dtype(dtype) && gate && up && act && M > 0 && I > 0 && ld >= I, W8A8_ERR_BAD_ARG);
    REQUIRE(M <= 65535, W8A8_ERR_UNSUPPORTED);
    REQUIRE(current_ready_device() >= 0, W8A8_ERR_NOT_INITIALIZED);
    CUDA_OK(launch_swiglu(gate, up, dtype, M, I, ld, act, maxima, (cudaStream_t)stream), "launch_swiglu");
    return W8A8_OK;
}

int w8a8_residual(const void *a, const void *b, int dtype, size_t n, void *out, void *stream) {
    REQUIRE(check_dtype(dtype) && a && b && out && n > 0, W8A8_ERR_BAD_ARG);
    REQUIRE(aligned16(a) && aligned16(b) && aligned16(out), W8A8_ERR_ALIGNMENT);
    REQUIRE(current_ready_device() >= 0, W8A8_ERR_NOT_INITIALIZED);
    CUDA_OK(launch_residual(a, b, dtype, n, out, (cudaStream_t)stream), "launch_residual");
    return W8A8_OK;
}

int w8a8_rounding_probe(const float *x, int8_t *out, size_t n, void *stream) {
    REQUIRE(x && out && n > 0, W8A8_ERR_BAD_ARG);
    REQUIRE(current_ready_device() >= 0, W8A8_ERR_NOT_INITIALIZED);
    CUDA_OK(launch_rounding_probe(x, out, n, (cudaStream_t)stream), "launch_rounding_probe");
    return W8A8_OK;
}

// ---- projections -----------------------------------------------------------------------

// Regime selection, from measurements on B200 (CUDA events, cold weights):
//   1 token            gemv_dp4a: whole weight rows per warp, 6.5 TB/s on the large projections
//   2..8 tokens        gemv_mma
//   9..16 tokens       gemm_skinny for the very large matrices (>= 256 MB), gemv_mma otherwise
//   17..64 tokens      gemm_skinny for the large matrices (>= 64 MB of weights), gemm_cluster otherwise
//   65..128 tokens     gemm_skinny for the very large ones (>= 256 MB), gemm_cluster for long-K matrices below 64 MB,
//                      gemm_tcgen05 otherwise
//   more               gemm_tcgen05_pair (256x256 tiles over CTA pairs); gemm_tcgen05 with 128- or 64-channel tiles
//                      while the pair kernel would have tiles for less than three quarters of the CTA pairs
static int pick_variant(int M, int epilogue, bool single_matrix, long long weight_bytes, int K) {
    if (M <= 1) return W8A8_VARIANT_GEMV_DP4A;
    if (epilogue == EPI_SWIGLU) return W8A8_VARIANT_GEMV_DP4A;  // fused gate/up exists only there (M <= 4)
    if (!single_matrix) return W8A8_VARIANT_GEMV_MMA;  // grouped siblings, 2..16 tokens
    if (M <= 8) return W8A8_VARIANT_GEMV_MMA;
    if (M <= 16) return weight_bytes >= (256ll << 20) ? W8A8_VARIANT_GEMM_SKINNY : W8A8_VARIANT_GEMV_MMA;
    // 17..64 tokens: the 16-50 MB matrices split K over a thread-block cluster (gemv_mma re-reads every token row per 16
    // channels: Q|K|V 25.6 -> 19.5 us, O 19.5 -> 15.4, down 29.7 -> 21.5 at 64 tokens, L2 displaced before every launch)
    if (M <= 64) return weight_bytes >= (64ll << 20) ? W8A8_VARIANT_GEMM_SKINNY : W8A8_VARIANT_GEMM_CLUSTER;
    if (M <= 128) {
        if (weight_bytes >= (256ll << 20)) return W8A8_VARIANT_GEMM_SKINNY;
        // long K, few channels (down): 23.6 us against 33.7 with 128-channel tiles on 32 SMs
        return (K >= 8192 && weight_bytes < (64ll << 20)) ? W8A8_VARIANT_GEMM_CLUSTER : W8A8_VARIANT_GEMM_TCGEN05;
    }
    // the same matrices up to 256 tokens: 24.6 / 28.7 / 32.8 us at 129 / 200 / 256 tokens against 34.8
    if (M <= kClusterMaxTokens && K >= 8192 && weight_bytes < (64ll << 20)) return W8A8_VARIANT_GEMM_CLUSTER;
    // 256x256 tiles over CTA pairs: 5-16 % faster than 128x256 tiles from 129 tokens up, as long as there are tiles
    // for most of the 74 pairs; otherwise (O, down, Q|K|V at a few hundred tokens) the single-CTA kernel, which then
    // narrows its tiles to 128 or 64 channels to put the matrix on more SMs.
    const long long N = weight_bytes / K;
    const int bn = pair_tile_channels(M, (int)N);
    const long long pair_tiles = ((M + 255) / 256) * ((N + bn - 1) / bn);
    if (pair_tiles * 4 < (long long)(sm_count() / 2) * 3) return W8A8_VARIANT_GEMM_TCGEN05;
    // Token counts just above a multiple of 256 (300 -> 512 padded rows against 384): the 128-row tiles do a quarter
    // less work, which outweighs the pair kernel's advantage per tile.
    if (((M + 255) / 256) * 256 * 100 > ((M + 127) / 128) * 128 * 115) return W8A8_VARIANT_GEMM_TCGEN05;
    return W8A8_VARIANT_GEMM_TCGEN05_PAIR;
}

static int run_linear(LinearArgs &l, const w8a8_weight *wt, int variant, void *stream) {
    REQUIRE(current_ready_device() >= 0, W8A8_ERR_NOT_INITIALIZED);
    if (variant == W8A8_VARIANT_AUTO)
        variant = pick_variant(l.M, l.epilogue, wt != nullptr && l.count == 1, (long long)l.n[0] * l.K, l.K);
    cudaStream_t s = (cudaStream_t)stream;
    switch (variant) {
        case W8A8_VARIANT_NAIVE: CUDA_OK(launch_linear_naive(l, s), "launch_linear_naive"); return W8A8_OK;
        case W8A8_VARIANT_GEMV_DP4A:
            REQUIRE(l.M <= 4 && l.K <= 24576, W8A8_ERR_UNSUPPORTED);
            CUDA_OK(launch_gemv_dp4a(l, s), "launch_gemv_dp4a");
            return W8A8_OK;
        case W8A8_VARIANT_GEMV_MMA:
            REQUIRE(l.M <= 64 && l.epilogue != EPI_SWIGLU, W8A8_ERR_UNSUPPORTED);
            CUDA_OK(launch_gemv_mma(l, s), "launch_gemv_mma");
            return W8A8_OK;
        case W8A8_VARIANT_GEMM_TCGEN05:
            REQUIRE(wt && l.count == 1 && l.epilogue != EPI_SWIGLU, W8A8_ERR_UNSUPPORTED);
            CUDA_OK(launch_gemm_tcgen05(l, wt, s), "launch_gemm_tcgen05");
            return W8A8_OK;
        case W8A8_VARIANT_GEMM_TCGEN05_PAIR:
            REQUIRE(wt && l.count == 1 && l.epilogue != EPI_SWIGLU, W8A8_ERR_UNSUPPORTED);
            CUDA_OK(launch_gemm_tcgen05_pair(l, wt, s), "launch_gemm_tcgen05_pair");
            return W8A8_OK;
        case W8A8_VARIANT_GEMM_CLUSTER:
            REQUIRE(wt && l.count == 1 && l.epilogue != EPI_SWIGLU && l.M <= kClusterMaxTokens, W8A8_ERR_UNSUPPORTED);
            CUDA_OK(launch_gemm_cluster(l, wt, s), "launch_gemm_cluster");
            return W8A8_OK;
        case W8A8_VARIANT_GEMM_SKINNY:
            REQUIRE(wt && l.count == 1 && l.epilogue != EPI_SWIGLU && l.M <= kSkinnyMaxTokens, W8A8_ERR_UNSUPPORTED);
            CUDA_OK(launch_gemm_skinny(l, wt, s), "launch_gemm_skinny");
            return W8A8_OK;
        default: return W8A8_ERR_BAD_ARG;
    }
}

static bool valid_weight(const w8a8_weight *w) { return w && w->magic == kWeightMagic; }

// The reference keeps every input and output of a projection in its own allocation (docs/qwen3-8b-w8a8/safety.md:15:
// residual, out and combined are three distinct buffers) and the kernels rely on it (weights and activations are read
// through the non-coherent path while outputs are written).  A byte range that an output shares with another operand
// is rejected here, on the host, before anything is queued.
struct ByteRange {
    const void *p;
    size_t n;
    const char *name;
};
static bool overlaps(const ByteRange &a, const ByteRange &b) {
    if (!a.p || !b.p || a.n == 0 || b.n == 0) return false;
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a.p), b0 = reinterpret_cast<uintptr_t>(b.p);
    return a0 < b0 + b.n && b0 < a0 + a.n;
}
// outputs[0 .. n_out) against each other and against inputs[0 .. n_in)
static int reject_aliasing(const ByteRange *outputs, int n_out, const ByteRange *inputs, int n_in, const char *where) {
    for (int i = 0; i < n_out; ++i) {
        for (int j = i + 1; j < n_out; ++j)
            if (overlaps(outputs[i], outputs[j])) {
                snprintf(g_err, sizeof g_err, "%s: outputs %s and %s overlap", where, outputs[i].name, outputs[j].name);
                return W8A8_ERR_BAD_ARG;
            }
        for (int j = 0; j < n_in; ++j)
            if (overlaps(outputs[i], inputs[j])) {
                snprintf(g_err, sizeof g_err, "%s: output %s overlaps input %s", where, outputs[i].name, inputs[j].name);
                return W8A8_ERR_BAD_ARG;
            }
    }
    return W8A8_OK;
}
static size_t elem_bytes(int dtype) { return dtype == W8A8_BF16 ? 2 : 4; }

int w8a8_linear_ex(const int8_t *q, const float *a_scale, w8a8_weight_t weight, int M, const void *residual, void *y,
                   void *combined, int dtype, int variant, void *stream) {
    REQUIRE(valid_weight(weight) && q && a_scale && M > 0 && check_dtype(dtype), W8A8_ERR_BAD_ARG);
    REQUIRE((residual == nullptr) == (combined == nullptr), W8A8_ERR_BAD_ARG);
    REQUIRE(y || combined, W8A8_ERR_BAD_ARG);
    REQUIRE(aligned16(q) && (y == nullptr || aligned16(y)) && (combined == nullptr || aligned16(combined)) &&
                (residual == nullptr || aligned16(residual)), W8A8_ERR_ALIGNMENT);
    {
        const size_t out_bytes = (size_t)M * weight->N * elem_bytes(dtype);
        const ByteRange outputs[] = {{y, out_bytes, "y"}, {combined, out_bytes, "combined"}};
        const ByteRange inputs[] = {{q, (size_t)M * weight->K, "q"}, {a_scale, (size_t)M * 4, "a_scale"},
                                    {weight->w, (size_t)weight->N * weight->K, "w"}, {weight->w_scale, (size_t)weight->N * 4, "w_scale"},
                                    {residual, out_bytes, "residual"}};
        const int st = reject_aliasing(outputs, 2, inputs, 5, "w8a8_linear");
        if (st != W8A8_OK) return st;
    }
    LinearArgs l{};
    l.q = q; l.a_scale = a_scale; l.M = M; l.K = weight->K; l.count = 1;
    l.w[0] = weight->w; l.ws[0] = weight->w_scale; l.out[0] = y; l.n[0] = weight->N;
    l.epilogue = residual ? EPI_RESIDUAL : EPI_PLAIN;
    l.residual = residual; l.combined = combined; l.dtype = dtype;
    return run_linear(l, weight, variant, stream);
}

int w8a8_linear(const int8_t *q, const float *a_scale, w8a8_weight_t weight, int M, const void *residual, void *y,
                void *combined, int dtype, void *stream) {
    return w8a8_linear_ex(q, a_scale, weight, M, residual, y, combined, dtype, W8A8_VARIANT_AUTO, stream);
}

int w8a8_linear_grouped(const int8_t *q, const float *a_scale, const w8a8_weight_t *weights, int count, int M,
                        void *const *outs, int dtype, void *stream) {
    REQUIRE(q && a_scale && weights && outs && count >= 1 && count <= kMaxGroup && M > 0 && check_dtype(dtype), W8A8_ERR_BAD_ARG);
    REQUIRE(M <= 16, W8A8_ERR_UNSUPPORTED);
    REQUIRE(aligned16(q), W8A8_ERR_ALIGNMENT);
    LinearArgs l{};
    l.q = q; l.a_scale = a_scale; l.M = M; l.count = count; l.epilogue = EPI_PLAIN; l.dtype = dtype;
    for (int g = 0; g < count; ++g) {
        REQUIRE(valid_weight(weights[g]) && outs[g], W8A8_ERR_BAD_ARG);
        REQUIRE(weights[g]->K == weights[0]->K, W8A8_ERR_BAD_ARG);
        REQUIRE(aligned16(outs[g]), W8A8_ERR_ALIGNMENT);
        l.w[g] = weights[g]->w; l.ws[g] = weights[g]->w_scale; l.out[g] = outs[g]; l.n[g] = weights[g]->N;
    }
    l.K = weights[0]->K;
    return run_linear(l, nullptr, W8A8_VARIANT_AUTO, stream);
}

int w8a8_linear_gate_up_swiglu(const int8_t *q, const float *a_scale, w8a8_weight_t w_gate, w8a8_weight_t w_up, int M,
                               void *gate_out, void *up_out, void *act, uint32_t *maxima, int dtype, void *stream) {
    REQUIRE(q && a_scale && valid_weight(w_gate) && valid_weight(w_up) && act && M > 0 && check_dtype(dtype), W8A8_ERR_BAD_ARG);
    REQUIRE(w_gate->K == w_up->K && w_gate->N == w_up->N, W8A8_ERR_BAD_ARG);
    REQUIRE(M <= 16, W8A8_ERR_UNSUPPORTED);
    REQUIRE(aligned16(q) && aligned16(act), W8A8_ERR_ALIGNMENT);
    LinearArgs l{};
    l.q = q; l.a_scale = a_scale; l.M = M; l.K = w_gate->K; l.count = 2; l.dtype = dtype;
    l.w[0] = w_gate->w; l.ws[0] = w_gate->w_scale; l.n[0] = w_gate->N; l.out[0] = gate_out;
    l.w[1] = w_up->w; l.ws[1] = w_up->w_scale; l.n[1] = w_up->N; l.out[1] = up_out;
    l.epilogue = EPI_SWIGLU; l.act = act; l.maxima = maxima;
    if (M <= 4) return run_linear(l, nullptr, W8A8_VARIANT_GEMV_DP4A, stream);
    // 5..16 tokens: the two projections in one grouped launch, then the element-wise SwiGLU.
    // The un-fused pair needs gate/up storage; the caller must supply both.
    REQUIRE(gate_out && up_out, W8A8_ERR_UNSUPPORTED);
    l.epilogue = EPI_PLAIN;
    int st = run_linear(l, nullptr, W8A8_VARIANT_GEMV_MMA, stream);
    if (st != W8A8_OK) return st;
    return w8a8_swiglu(gate_out, up_out, dtype, M, w_gate->N, w_gate->N, act, maxima, stream);
}

// One-token projections with the activation quantizer in the GEMV's prologue (gemv.cu: quantize_prologue).
static int fused_source(LinearArgs &l, const void *x, int dtype, int source, const void *gamma, float eps,
                        const uint32_t *maxima_in, uint32_t *maxima_reset, int reset_words, int8_t *q_out, float *scale_out) {
    REQUIRE(x && check_dtype(dtype), W8A8_ERR_BAD_ARG);
    REQUIRE(source == W8A8_SOURCE_WITH_MAX || source == W8A8_SOURCE_RMSNORM, W8A8_ERR_BAD_ARG);
    REQUIRE(source != W8A8_SOURCE_WITH_MAX || maxima_in, W8A8_ERR_BAD_ARG);
    REQUIRE(source != W8A8_SOURCE_RMSNORM || gamma, W8A8_ERR_BAD_ARG);
    REQUIRE(reset_words >= 0 && reset_words <= 8 && (reset_words == 0 || maxima_reset), W8A8_ERR_BAD_ARG);
    REQUIRE(aligned16(x) && (gamma == nullptr || aligned16(gamma)) && (q_out == nullptr || aligned16(q_out)), W8A8_ERR_ALIGNMENT);
    REQUIRE(l.K <= (source == W8A8_SOURCE_RMSNORM ? 16384 : 24576), W8A8_ERR_UNSUPPORTED);
    l.M = 1; l.dtype = dtype;
    l.src = source == W8A8_SOURCE_WITH_MAX ? SRC_WITH_MAX : SRC_RMSNORM;
    l.x = x; l.gamma = gamma; l.eps = eps; l.maxima_in = maxima_in; l.maxima_reset = maxima_reset; l.reset_words = reset_words;
    l.q_out = q_out; l.scale_out = scale_out;
    return W8A8_OK;
}

int w8a8_quantize_linear(const void *x, int dtype, int source, const void *gamma, float eps, const uint32_t *maxima_in,
                         w8a8_weight_t weight, const void *residual, void *y, void *combined, uint32_t *maxima_reset,
                         int reset_words, int8_t *q_out, float *scale_out, void *stream) {
    REQUIRE(valid_weight(weight), W8A8_ERR_BAD_ARG);
    REQUIRE((residual == nullptr) == (combined == nullptr) && (y || combined), W8A8_ERR_BAD_ARG);
    REQUIRE((y == nullptr || aligned16(y)) && (combined == nullptr || aligned16(combined)) && (residual == nullptr || aligned16(residual)),
            W8A8_ERR_ALIGNMENT);
    LinearArgs l{};
    l.K = weight->K; l.count = 1;
    l.w[0] = weight->w; l.ws[0] = weight->w_scale; l.out[0] = y; l.n[0] = weight->N;
    l.epilogue = residual ? EPI_RESIDUAL : EPI_PLAIN;
    l.residual = residual; l.combined = combined;
    const int st = fused_source(l, x, dtype, source, gamma, eps, maxima_in, maxima_reset, reset_words, q_out, scale_out);
    if (st != W8A8_OK) return st;
    return run_linear(l, weight, W8A8_VARIANT_GEMV_DP4A, stream);
}

int w8a8_quantize_linear_gate_up_swiglu(const void *x, int dtype, int source, const void *gamma, float eps,
                                        const uint32_t *maxima_in, w8a8_weight_t w_gate, w8a8_weight_t w_up, void *act,
                                        uint32_t *maxima_out, int8_t *q_out, float *scale_out, void *stream) {
    REQUIRE(valid_weight(w_gate) && valid_weight(w_up) && act, W8A8_ERR_BAD_ARG);
    REQUIRE(w_gate->K == w_up->K && w_gate->N == w_up->N, W8A8_ERR_BAD_ARG);
    REQUIRE(aligned16(act), W8A8_ERR_ALIGNMENT);
    LinearArgs l{};
    l.K = w_gate->K; l.count = 2;
    l.w[0] = w_gate->w; l.ws[0] = w_gate->w_scale; l.n[0] = w_gate->N;
    l.w[1] = w_up->w; l.ws[1] = w_up->w_scale; l.n[1] = w_up->N;
    l.epilogue = EPI_SWIGLU; l.act = act; l.maxima = maxima_out;
    const int st = fused_source(l, x, dtype, source, gamma, eps, maxima_in, nullptr, 0, q_out, scale_out);
    if (st != W8A8_OK) return st;
    return run_linear(l, nullptr, W8A8_VARIANT_GEMV_DP4A, stream);
}

int w8a8_linear_no_alloc(const int8_t *q, const float *a_scale, const int8_t *w, const float *w_scale, int M, int N, int K,
                         void *y, int dtype, void *stream) {
    REQUIRE(q && a_scale && w && w_scale && y && M > 0 && N > 0 && K > 0 && check_dtype(dtype), W8A8_ERR_BAD_ARG);
    REQUIRE(K % 128 == 0 && aligned16(q) && aligned16(y) && (reinterpret_cast<uintptr_t>(w) & 127u) == 0 && aligned16(w_scale),
            W8A8_ERR_ALIGNMENT);
    {
        const ByteRange outputs[] = {{y, (size_t)M * N * elem_bytes(dtype), "y"}};
        const ByteRange inputs[] = {{q, (size_t)M * K, "q"}, {a_scale, (size_t)M * 4, "a_scale"}, {w, (size_t)N * K, "w"},
                                    {w_scale, (size_t)N * 4, "w_scale"}};
        const int st = reject_aliasing(outputs, 1, inputs, 4, "w8a8_linear_no_alloc");
        if (st != W8A8_OK) return st;
    }
    if (M > kNoAllocMaxTokens) {
        snprintf(g_err, sizeof g_err, "w8a8_linear_no_alloc: M=%d exceeds the %d tokens its fixed scratch array holds", M,
                 kNoAllocMaxTokens);
        return W8A8_ERR_UNSUPPORTED;
    }
    CUDA_OK(launch_linear_no_alloc(q, a_scale, w, w_scale, M, N, K, y, dtype, (cudaStream_t)stream), "launch_linear_no_alloc");
    return W8A8_OK;
}

int w8a8_linear_argmax(const int8_t *q, const float *a_scale, w8a8_weight_t weight, int M, uint32_t *token, float *value,
                       void *stream) {
    REQUIRE(valid_weight(weight) && q && a_scale && token && M > 0, W8A8_ERR_BAD_ARG);
    REQUIRE(aligned16(q), W8A8_ERR_ALIGNMENT);
    REQUIRE(M <= 16 && (weight->N + 15) / 16 <= kArgmaxMaxBlocks, W8A8_ERR_UNSUPPORTED);
    REQUIRE(current_ready_device() >= 0, W8A8_ERR_NOT_INITIALIZED);
    LinearArgs l{};
    l.q = q; l.a_scale = a_scale; l.M = M; l.K = weight->K; l.count = 1; l.dtype = W8A8_BF16;
    l.w[0] = weight->w; l.ws[0] = weight->w_scale; l.n[0] = weight->N;
    l.epilogue = EPI_ARGMAX; l.partial_best = argmax_scratch();
    cudaStream_t s = (cudaStream_t)stream;
    CUDA_OK(launch_gemv_mma(l, s), "launch_gemv_mma(argmax)");
    CUDA_OK(launch_argmax_finish(l.partial_best, (weight->N + 15) / 16, M, token, value, s), "launch_argmax_finish");
    return W8A8_OK;
}

int w8a8_linear_allreduce(const int8_t *q, const float *a_scale, w8a8_weight_t weight, int M, const void *residual, void *y,
                          void *combined, int dtype, void *const *peer_packets, uint32_t *seq, int rank, int tp,
                          size_t slot_packets, void *stream) {
    REQUIRE(valid_weight(weight) && q && a_scale && M > 0 && check_dtype(dtype), W8A8_ERR_BAD_ARG);
    REQUIRE(peer_packets && seq && tp >= 1 && tp <= kTpMaxRanks && rank >= 0 && rank < tp, W8A8_ERR_BAD_ARG);
    REQUIRE((residual == nullptr) == (combined == nullptr) && (y || combined), W8A8_ERR_BAD_ARG);
    REQUIRE(M <= 64 && (size_t)M * weight->N <= slot_packets, W8A8_ERR_UNSUPPORTED);
    REQUIRE(aligned16(q), W8A8_ERR_ALIGNMENT);
    LinearArgs l{};
    l.q = q; l.a_scale = a_scale; l.M = M; l.K = weight->K; l.count = 1;
    l.w[0] = weight->w; l.ws[0] = weight->w_scale; l.n[0] = weight->N;
    l.epilogue = EPI_PUSH; l.dtype = dtype;
    for (int p = 0; p < tp; ++p) {
        REQUIRE(peer_packets[p] && (reinterpret_cast<uintptr_t>(peer_packets[p]) & 7u) == 0, W8A8_ERR_ALIGNMENT);
        l.push.ll[p] = static_cast<uint2 *>(peer_packets[p]);
    }
    l.push.seq = seq; l.push.rank = rank; l.push.tp = tp; l.push.slot = slot_packets;
    const int st = run_linear(l, weight, M == 1 ? W8A8_VARIANT_GEMV_DP4A : W8A8_VARIANT_GEMV_MMA, stream);
    if (st != W8A8_OK) return st;
    CUDA_OK(launch_tp_reduce(static_cast<const uint2 *>(peer_packets[rank]), seq, residual, y, combined, (size_t)M * weight->N, dtype, tp,
                             slot_packets, (cudaStream_t)stream),
            "launch_tp_reduce");
    return W8A8_OK;
}

int w8a8_tp_allreduce(const void *partial, void *out, size_t n_el, int dtype, void *const *peer_bufs, uint32_t *const *peer_flags,
                      uint32_t *seq, int rank, int tp, size_t slot_el, void *stream) {
    REQUIRE(partial && out && peer_bufs && peer_flags && seq && check_dtype(dtype), W8A8_ERR_BAD_ARG);
    REQUIRE(tp >= 1 && tp <= 8 && rank >= 0 && rank < tp && n_el > 0 && n_el <= slot_el, W8A8_ERR_BAD_ARG);
    REQUIRE(n_el % elem_vec(dtype) == 0 && slot_el % elem_vec(dtype) == 0 && aligned16(partial) && aligned16(out), W8A8_ERR_ALIGNMENT);
    for (int p = 0; p < tp; ++p) REQUIRE(peer_bufs[p] && peer_flags[p] && aligned16(peer_bufs[p]), W8A8_ERR_BAD_ARG);
    REQUIRE(current_ready_device() >= 0, W8A8_ERR_NOT_INITIALIZED);
    CUDA_OK(launch_tp_allreduce(partial, out, n_el, dtype, peer_bufs, peer_flags, seq, rank, tp, slot_el, (cudaStream_t)stream),
            "launch_tp_allreduce");
    return W8A8_OK;
}

int w8a8_linear_acc_i32(const int8_t *q, w8a8_weight_t weight, int M, int32_t *acc, int variant, void *stream) {
    REQUIRE(valid_weight(weight) && q && acc && M > 0, W8A8_ERR_BAD_ARG);
    REQUIRE(aligned16(q) && aligned16(acc), W8A8_ERR_ALIGNMENT);
    LinearArgs l{};
    l.q = q; l.M = M; l.K = weight->K; l.count = 1; l.dtype = W8A8_BF16;
    l.w[0] = weight->w; l.ws[0] = weight->w_scale; l.n[0] = weight->N;
    l.epilogue = EPI_ACC; l.acc = acc;
    return run_linear(l, weight, variant, stream);
}

}  // extern "C"
