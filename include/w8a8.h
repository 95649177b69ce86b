/*
 * w8a8.h -- C ABI of the B200 (sm_100a) W8A8 linear-layer library.
 *
 * The library stands where the inferrous-qwen3 host runtime calls the kernel
 * launchers that its `#[cuda_module]` macro generates (src/kernels.rs:322-323,
 * invoked as `module.KERNEL(&stream, LaunchConfig, args...)`, e.g. src/gpu.rs:351-360).
 * Each entry point below names the reference launcher(s) it replaces.
 *
 * Conventions (they restate the reference's own, docs/qwen3-8b-w8a8/safety.md):
 *  - every pointer is a DEVICE pointer owned by the caller unless stated otherwise;
 *    inputs and outputs never alias; all buffers outlive the queued work;
 *  - `stream` is a cudaStream_t / CUstream passed as void*; all work is queued on
 *    it, nothing synchronises, nothing touches the default stream;
 *  - launch calls allocate nothing, read no device memory from the host and are
 *    safe inside stream capture once w8a8_init() has run for the device;
 *  - every kernel executes `griddepcontrol.wait` before its first access to a
 *    buffer another kernel may produce, so programmatic graph edges
 *    (src/graph.rs:63-127, src/kernels.rs:173-184) stay legal;
 *  - activations are row-major [M,K]; weights are row-major [N,K] int8 (K contiguous)
 *    with one f32 scale per output channel; outputs are row-major [M,N];
 *  - activation element type is selectable: W8A8_BF16 (2-byte storage) or W8A8_F32
 *    (the reference's carrier: f32 buffers that hold bf16-representable values,
 *    src/gpu.rs:16).  Results are the same values in either carrier;
 *  - every function returns a w8a8_status_t; nothing throws, traps or aborts.
 */
#ifndef W8A8_H
#define W8A8_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    W8A8_OK = 0,
    W8A8_ERR_BAD_ARG = 1,      /* null pointer, non-positive size, unknown enum */
    W8A8_ERR_ALIGNMENT = 2,    /* K not a multiple of 128, pointer not 16-byte aligned */
    W8A8_ERR_UNSUPPORTED = 3,  /* shape outside what the chosen kernel variant handles */
    W8A8_ERR_CUDA = 4,         /* a CUDA runtime/driver call failed; see w8a8_last_cuda_error */
    W8A8_ERR_DEVICE_TIMEOUT = 5, /* a bounded device-side wait expired (reported by w8a8_device_status) */
    W8A8_ERR_NOT_INITIALIZED = 6 /* w8a8_init() has not run for the current device */
} w8a8_status_t;

typedef enum { W8A8_BF16 = 0, W8A8_F32 = 1 } w8a8_dtype_t;

/* Kernel selection for w8a8_linear_ex.  AUTO is what w8a8_linear uses and mirrors the
 * regime switch of GpuModel::linear_quantized (src/gpu.rs:450-509). */
typedef enum {
    W8A8_VARIANT_AUTO = 0,
    W8A8_VARIANT_NAIVE = 1,      /* one thread per output; the on-GPU oracle (role of `linear`, src/kernels.rs:808-845) */
    W8A8_VARIANT_GEMV_DP4A = 2,  /* M <= 4: 16-byte weight streaming + dp4a + in-CTA split-K */
    W8A8_VARIANT_GEMV_MMA = 3,   /* M <= 64: 16-byte weight streaming + warp-level int8 MMA */
    W8A8_VARIANT_GEMM_TCGEN05 = 4, /* any M: TMA-staged 128x256 tiles + tcgen05.mma kind::i8 into TMEM */
    W8A8_VARIANT_GEMM_SKINNY = 5,  /* M <= 256: tcgen05 with the weights on the MMA's M side, stream-K split */
    /* 6 and 7 named two kernels that lost to the others on every shape and were removed; the values stay unused */
    W8A8_VARIANT_GEMM_TCGEN05_PAIR = 8, /* any M: 256x256 tiles over CTA pairs (tcgen05.mma.cta_group::2) */
    W8A8_VARIANT_GEMM_CLUSTER = 9       /* M <= 256: tcgen05, weights on the MMA's M side, K split over a thread-block
                                           cluster with the partial sums reduced through distributed shared memory */
} w8a8_variant_t;

/* Immutable weight matrix handle: device pointers, shape and the TMA descriptor of the
 * [N,K] matrix (replaces gpu::Matrix{w,map,scale,k,n}, src/gpu.rs:43-49, and
 * tensor::map, src/tensor.rs:5-39). */
typedef struct w8a8_weight *w8a8_weight_t;

/* ---- library / device set-up -------------------------------------------------------- */

/* Loads kernels and sets their attributes on `device` (replaces device::load(&ctx),
 * src/gpu.rs:250).  Call once per device before any launch and before stream capture. */
int w8a8_init(int device);
/* Library version, "major.minor.patch". */
const char *w8a8_version(void);
const char *w8a8_status_string(int status);
/* Text of the last failing CUDA call on this host thread ("" if none). */
const char *w8a8_last_cuda_error(void);
/* Next-weight L2 prefetch (the role of the reference's prefetch CTAs and row tables, src/kernels.rs:173-237,
 * src/gpu.rs:19-42): registers [weights, weights + bytes) -- device memory that no kernel writes, normally int8 rows
 * of a projection that runs a few launches later -- with the calling thread; up to four ranges may be pending.  The
 * next qwen3_attention launch, or quantizer launch (w8a8_quantize, w8a8_quantize_with_max, w8a8_rmsnorm_quantize,
 * w8a8_swiglu_quantize) of at most 16 rows, from that thread carries one extra CTA per SM that issues
 * `prefetch.global.L2` for those lines and leaves.  The hints are consumed by that launch (inside a stream capture they become part of the captured
 * kernel node).  A hint only moves data towards L2 earlier; results never depend on it.  (NULL, 0) clears the list. */
int w8a8_prefetch_hint(const void *weights, size_t bytes);

/* Programmatic dependent launch, the reference's CLEAN_PDL switch (src/gpu.rs:317; the graph rewrite of
 * src/graph.rs:63-127).  When enabled (default off; env W8A8_PDL=1 at init), every hot-path kernel is
 * launched with the programmatic-stream-serialization attribute: it may begin while its predecessor on
 * the stream drains, and its own griddepcontrol.wait orders the data.  Captured into a CUDA graph the
 * launches become programmatic edges.  Process-wide switch; set it before capturing. */
int w8a8_set_programmatic_launch(int enabled);
/* Reads (and clears) the device-side status words of the current device: 0, or
 * W8A8_ERR_DEVICE_TIMEOUT with *detail = code of the wait that gave up (code << 24 | low bits of its argument).
 * Codes: 1-4 a stage of a TMA / tensor-core pipeline, 5 another rank's partial outputs (tensor parallel), 6 a token id
 * or cache position out of range (not a wait: the access was skipped), 7 a grid-wide barrier of qwen3_decode_layers.
 * Synchronises `stream`.  It covers both the status word w8a8_init() allocated and the one inside the fixed array of
 * w8a8_linear_no_alloc, so it also works on a device where only that entry point has run.  Scratch that launches
 * share and leave at zero (stream-K partial tiles and arrival counters of w8a8_linear for 9..128 tokens, the
 * key-split counters of qwen3_attention) may be left dirty by a launch whose wait ran out; when this call finds
 * such a code it returns that scratch to zero in stream order, so that the launches which follow are right again.
 * Until then results on that device are undefined: after a device timeout, call this before anything else.
 * That scratch is per device, not per stream: launches of w8a8_linear (9..128 tokens), w8a8_linear_argmax and
 * qwen3_attention on different streams of one device must not overlap on the GPU. */
int w8a8_device_status(void *stream, uint32_t *detail);

/* ---- weights ------------------------------------------------------------------------ */

/* Wraps caller-owned device buffers w[N,K] int8 and w_scale[N] f32.  No copy is made.
 * Replaces the Matrix construction at src/gpu.rs:258-299.  K % 128 == 0, w 128-byte aligned. */
int w8a8_weight_create(const int8_t *w, const float *w_scale, int N, int K, w8a8_weight_t *out);
int w8a8_weight_destroy(w8a8_weight_t weight);
int w8a8_weight_shape(w8a8_weight_t weight, int *N, int *K);

/* Bytes of the hot path's share of the reference's Workspace (src/gpu.rs:76-143) for launches of up to `max_rows` rows:
 * the int8 codes of the three activation widths (hidden, q_width = query heads x 128, intermediate), one f32 scale and
 * one u32 absolute-maximum word per row, each region rounded up to 256 bytes, in that order.  `offsets` (optional, 5
 * entries) receives the byte offset of each region in a single allocation of that size: codes[hidden], codes[q_width],
 * codes[intermediate], scales, maxima.  Host arithmetic only: no CUDA call, no w8a8_init() needed.  0 on a non-positive
 * argument. */
size_t w8a8_workspace_bytes(int max_rows, int hidden, int q_width, int intermediate, size_t *offsets);

/* ---- activation quantizers ---------------------------------------------------------- */

/* `quantize` (src/kernels.rs:415-452; host wrapper src/gpu.rs:424-449):
 * scale[m] = max(1e-8, max_k |x[m,k]|) / 127;  q[m,k] = rne(clamp(x[m,k] / scale[m], +-127)).
 * ldx = row stride of x in elements (>= K). */
int w8a8_quantize(const void *x, int dtype, int M, int K, int64_t ldx, int8_t *q, float *scale,
                  void *stream);

/* `quantize_with_max` (src/kernels.rs:455-475; src/gpu.rs:377-390): the row maximum is
 * given as f32 bit patterns, maxima[m] (as produced by the swiglu entry points). */
int w8a8_quantize_with_max(const void *x, int dtype, const uint32_t *maxima, int M, int K, int64_t ldx,
                           int8_t *q, float *scale, void *stream);

/* `norm_quantize` (src/kernels.rs:479-576; src/gpu.rs:340-363), any K % 128 == 0:
 * y = bf16((x * rsqrt(mean(x^2) + eps)) * gamma), then quantize(y).  gamma has the same
 * element type as x.  y_out (optional, may be NULL) receives the bf16 row the codes were
 * made from; maxima_reset (optional) gets 1e-8f bits per row, as the reference resets
 * the SwiGLU maximum there (src/kernels.rs:566). */
int w8a8_rmsnorm_quantize(const void *x, const void *gamma, int dtype, float eps, int M, int K, int64_t ldx,
                          int8_t *q, float *scale, void *y_out, uint32_t *maxima_reset, void *stream);

/* `swiglu` (src/kernels.rs:2172-2190; src/gpu.rs:768-778): act = bf16((g / (1 + exp(-g))) * u).
 * gate/up are [M,I] with row stride ld (elements); a [M,2I] gate|up buffer is passed as
 * gate = base, up = base + I, ld = 2I.  maxima (optional): atomic max of |act| bit patterns per row;
 * the caller resets it (w8a8_rmsnorm_quantize does). */
int w8a8_swiglu(const void *gate, const void *up, int dtype, int M, int I, int64_t ld, void *act,
                uint32_t *maxima, void *stream);

/* SwiGLU fused with the quantizer of the down-projection input (replaces the prefill pair
 * `swiglu` + `quantize`, src/gpu.rs:768-778 + :377-398).  act_out is optional. */
int w8a8_swiglu_quantize(const void *gate, const void *up, int dtype, int M, int I, int64_t ld, int8_t *q,
                         float *scale, void *act_out, void *stream);

/* `residual` (src/kernels.rs:2163-2170; src/gpu.rs:510-517): out = bf16(a + b), n elements. */
int w8a8_residual(const void *a, const void *b, int dtype, size_t n, void *out, void *stream);

/* ---- the W8A8 product + dequantizing epilogue --------------------------------------- */

/* GpuModel::linear_quantized / linear_residual (src/gpu.rs:450-509, :364-423), i.e. the kernels
 * `linear`, `linear_splitk`, `linear_tiled`, `linear_large`, `linear_residual`, `residual`:
 *   acc[m,n] = sum_k q[m,k] * w[n,k]            (int32, exact)
 *   y[m,n]   = bf16((f32(acc) * a_scale[m]) * w_scale[n])
 *   combined[m,n] = bf16(residual[m,n] + y[m,n])   when residual != NULL
 * y may be NULL when combined is requested and the un-summed projection is not needed.
 * The regime (decode GEMV / tensor-core GEMM) is chosen from M.
 * Operands must not share memory (docs/qwen3-8b-w8a8/safety.md:15: residual, out and combined are three distinct
 * buffers): a byte range that y or combined shares with each other or with q, a_scale, the weights, their scales or
 * residual is rejected with W8A8_ERR_BAD_ARG (the pair is named in w8a8_last_cuda_error()) before anything is queued. */
int w8a8_linear(const int8_t *q, const float *a_scale, w8a8_weight_t weight, int M, const void *residual,
                void *y, void *combined, int dtype, void *stream);
/* Same with an explicit kernel variant (tests: every variant must equal the naive one). */
int w8a8_linear_ex(const int8_t *q, const float *a_scale, w8a8_weight_t weight, int M, const void *residual,
                   void *y, void *combined, int dtype, int variant, void *stream);

/* `linear_pair` / `linear_triple` (src/kernels.rs:698-806; src/gpu.rs:571-590): up to three
 * sibling projections of the same quantized activations in one launch (Q, K, V).
 * All weights share K.  M <= 16. */
int w8a8_linear_grouped(const int8_t *q, const float *a_scale, const w8a8_weight_t *weights, int count, int M,
                        void *const *outs, int dtype, void *stream);

/* `linear_swiglu` (src/kernels.rs:621-695; src/gpu.rs:730-745): gate and up projections that
 * share every activation load, then act = bf16(silu(bf16 g) * bf16 u) and an atomic max of
 * |act| bit patterns into maxima[m].  gate_out / up_out are optional.  M <= 16. */
int w8a8_linear_gate_up_swiglu(const int8_t *q, const float *a_scale, w8a8_weight_t w_gate, w8a8_weight_t w_up,
                               int M, void *gate_out, void *up_out, void *act, uint32_t *maxima, int dtype,
                               void *stream);

/* One-token (decode) projections with the activation quantizer folded into the projection kernel: every CTA
 * quantizes the row for itself while its first weight loads are in flight, so no quantizer kernel runs between the
 * producer of the row and the projection.  Each call replaces a pair of reference launches at M = 1:
 *   W8A8_SOURCE_RMSNORM   `norm_quantize` (src/kernels.rs:479-576; GpuModel::norm_quantize, src/gpu.rs:340-363)
 *   W8A8_SOURCE_WITH_MAX  `quantize_with_max` (src/kernels.rs:455-475; src/gpu.rs:377-390): maxima_in[0] holds the bit
 *                         pattern of max(1e-8, max|x|), published by the producer of x with an atomic max
 * followed by `linear` / `linear_residual` (w8a8_quantize_linear) or `linear_swiglu`
 * (w8a8_quantize_linear_gate_up_swiglu).  Codes, scale and outputs are bit-identical to running the two entry
 * points one after the other; the reference itself has no fused form of these pairs.
 * x is one row of K elements.  Optional outputs written by the first CTA: `q_out` ([K] codes) and `scale_out` ([1]).
 * `maxima_reset`: `reset_words` (<= 8) words set to the bits of 1e-8f, the state an atomic-max consumer starts from
 * (the side effect GpuModel::norm_quantize has on its `maxima` argument); they must not be words that a kernel
 * between this call's predecessor and its successor still reads.  K <= 16384 (RMSNORM) / 24576 (WITH_MAX). */
#define W8A8_SOURCE_WITH_MAX 1
#define W8A8_SOURCE_RMSNORM 2
int w8a8_quantize_linear(const void *x, int dtype, int source, const void *gamma, float eps, const uint32_t *maxima_in,
                         w8a8_weight_t weight, const void *residual, void *y, void *combined, uint32_t *maxima_reset,
                         int reset_words, int8_t *q_out, float *scale_out, void *stream);
int w8a8_quantize_linear_gate_up_swiglu(const void *x, int dtype, int source, const void *gamma, float eps,
                                        const uint32_t *maxima_in, w8a8_weight_t w_gate, w8a8_weight_t w_up, void *act,
                                        uint32_t *maxima_out, int8_t *q_out, float *scale_out, void *stream);

/* The same projection, y = bf16((f32(acc) * a_scale[m]) * w_scale[n]), for callers that must not
 * allocate device memory: code running where cudaMalloc is forbidden or unavailable -- inside a
 * stream capture that the host application owns, in a process whose memory pool is closed after
 * start-up, or in a plug-in that is handed buffers and a stream and nothing else.  It needs neither
 * w8a8_init nor a weight handle (both allocate): weights are passed as raw pointers, and the
 * partial-sum tiles that the stream-K kernel exchanges between CTAs live in a fixed 1.25 MiB device
 * array inside the library (held by every GPU that loads the library until the process exits).
 * There is no counterpart in the reference; it is an addition of this library.
 * Limits: M <= 16 tokens (W8A8_ERR_UNSUPPORTED beyond, with the reason in w8a8_last_cuda_error()),
 * plain epilogue only.  The first call on a device resolves the array's address and raises the
 * kernel's shared-memory limit (host threads may race for that first call; it is done under a lock);
 * make that first call before any stream capture.  Every call clears the array's partial tiles and
 * counters in stream order and then uses them, so two calls that overlap on the GPU (different
 * streams, or a captured graph replayed concurrently with itself) race on it: keep them in order.
 * A bounded device-side wait that runs out leaves y undefined and its code in two status words of
 * the same array, which calls do NOT clear: w8a8_device_status reports and clears them (it needs no
 * w8a8_init for that). */
int w8a8_linear_no_alloc(const int8_t *q, const float *a_scale, const int8_t *w, const float *w_scale, int M, int N,
                         int K, void *y, int dtype, void *stream);

/* Head projection with greedy token selection fused into its epilogue: token[m] = argmax_n of
 * y[m,n] = bf16((f32(acc) * a_scale[m]) * w_scale[n]) without ever storing the logits.  Selection follows
 * `select_token` (src/kernels.rs:2191-2231; host check model::argmax, src/model.rs:206-218): the largest value wins,
 * equal values (0.0 and -0.0 included) go to the lowest index, and a row with any non-finite logit yields 0xffffffff.
 * value (optional) receives the winning logit.  Replaces the pair `head` + `select_token` (src/gpu.rs:801-811) for a
 * W8A8 head; the reference's own head is bf16 weights (src/kernels.rs:2233-2373).  M <= 16, N <= 262144.
 * Calls on different streams share one per-device candidate buffer: keep them in order. */
int w8a8_linear_argmax(const int8_t *q, const float *a_scale, w8a8_weight_t weight, int M, uint32_t *token, float *value,
                       void *stream);

/* Row-split projection (O, down) under tensor parallelism with its all-reduce fused in, for decode-sized launches
 * (M <= 64); no counterpart in the reference, which is single-GPU.  Two kernels per call and rank, no library collective:
 *   1. the weight-streaming GEMV of w8a8_linear, whose epilogue, instead of writing its partial output, sends every
 *      value to the same slot of EVERY rank as one 8-byte packet {float32 bits of the bf16 value, tag of this call} --
 *      a single peer store, so value and tag arrive together and no fence or flag write follows;
 *   2. a consumer that waits (bounded, about 2 s) until the tp packets of an element carry this call's tag, adds them in
 *      rank order in float32, rounds to bf16 (= y) and adds the residual (combined = bf16(residual + y)) -- the
 *      epilogue of `linear_residual`, with the sum over ranks in between; identical on every rank.
 *   peer_packets[p]  packet buffer of rank p as seen from this GPU: 2 * tp * slot_packets packets of 8 bytes, zero
 *                    before the first call (two halves used alternately, so nothing is cleared between calls)
 *   seq              2 uint32 in local memory, zero before the first call (completed calls, CTAs done), kept by the kernels
 * Every rank must issue the same sequence of calls with the same M and N (M * N <= slot_packets).  An expired wait is
 * reported by w8a8_device_status.  Only plain stores and loads touch peer memory. */
int w8a8_linear_allreduce(const int8_t *q, const float *a_scale, w8a8_weight_t weight, int M, const void *residual, void *y,
                          void *combined, int dtype, void *const *peer_packets, uint32_t *seq, int rank, int tp,
                          size_t slot_packets, void *stream);

/* Tensor-parallel sum of the row-split projections' partial outputs (O, down) over peer memory; no counterpart in
 * the reference, which is single-GPU.  One kernel per rank pushes the local partial into every rank's staging buffer
 * with plain peer stores, waits (bounded) for the other ranks' pushes and writes out = bf16(sum over ranks, in rank
 * order, accumulated in f32) -- identical on every rank.
 *   peer_bufs[p]   staging buffer of rank p, visible from this GPU: 2 * tp * slot_el elements
 *   peer_flags[p]  flag pad of rank p: tp uint32 counters, zero before the first call
 *   seq            4 uint32 in local memory, zero before the first call (call number and CTA counts, kept by the kernel)
 * Every rank must issue the same sequence of calls with the same n_el.  An expired wait is reported by
 * w8a8_device_status.  Meant for decode-sized messages (n_el <= slot_el). */
int w8a8_tp_allreduce(const void *partial, void *out, size_t n_el, int dtype, void *const *peer_bufs,
                      uint32_t *const *peer_flags, uint32_t *seq, int rank, int tp, size_t slot_el, void *stream);

/* Raw int32 accumulators acc[M,N] of the product (debug / parity: the reference's tests
 * hold these bit-exact through its CPU-integer fixtures, tools/operator_fixtures.py:54). */
int w8a8_linear_acc_i32(const int8_t *q, w8a8_weight_t weight, int M, int32_t *acc, int variant, void *stream);

/* `rounding_probe` (src/kernels.rs:326-333): out[i] = rne(clamp(x[i], +-127)) as int8. */
int w8a8_rounding_probe(const float *x, int8_t *out, size_t n, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* W8A8_H */
