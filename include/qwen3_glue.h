/* C ABI of the three operators that surround the W8A8 linear layers inside one Qwen3 decoder layer, so that a
 * host can run a whole forward pass through libw8a8.so: token embedding, per-head RMSNorm + rotary embedding +
 * KV-cache append, and causal grouped-query attention.  They are the callers on either side of the linear-layer
 * path declared in w8a8.h, not part of it: kernels that restate the reference's arithmetic.  Embedding, head
 * norm and rotary embedding keep the reference's summation order (bit-identical but for rsqrt.approx); attention
 * reassociates its float32 sums for parallelism (and runs its two products on the tensor cores from 32 rows up) and
 * stays within the reference's own tolerance for that operator.
 *
 * Reference interfaces replaced (paths under crates/inferrous-qwen3/):
 *   qwen3_embedding    kernel `embedding`   src/kernels.rs:335-345   launched at src/gpu.rs:543-551
 *   qwen3_prepare_qk   kernel `prepare_qk`  src/kernels.rs:1350-1443 launched at src/gpu.rs:626-641
 *   qwen3_attention    kernel `attention`   src/kernels.rs:1490-1658 launched at src/gpu.rs:659-671
 *                      (`attention_prefill` :1664 and the three-kernel long-context form :1832-2160 compute the
 *                      same function with other launch shapes; one kernel serves every length here)
 *
 * Conventions are those of w8a8.h: device pointers, work queued on `stream`, nothing synchronises or allocates,
 * int status return (W8A8_OK = 0), w8a8_init() first.  `dtype` is the activation carrier (W8A8_BF16 / W8A8_F32).
 * Head width is 128, the context at most 4096 positions (src/lib.rs:16-18).
 *
 * `control` is the reference's two-word device buffer {token id, absolute position of the first row}
 * (src/gpu.rs:189); the position is read on the device so that a captured graph can be replayed for every step.
 * qwen3_prepare_qk and qwen3_attention read the position BEFORE their programmatic-launch dependency wait (it decides
 * which cache lines they prefetch): when kernels are launched with programmatic edges, `control` must have been written
 * by an operation that completed before the PRECEDING kernel started -- the host upload the reference does before each
 * step qualifies; a kernel launched immediately before them that writes `control` does not.
 * A position or token id beyond its limit is not an error the host can see at launch time: the kernel skips the
 * access and records code 6 in the device status word (w8a8_device_status).
 *
 * KV caches: `k_cache` and `v_cache` are [capacity][kv_heads][128] bf16, token-major, owned by the caller.  The
 * layout is private to qwen3_prepare_qk and qwen3_attention (the reference stores its keys channel-major).
 */
#ifndef QWEN3_GLUE_H
#define QWEN3_GLUE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* out[r, :] = table[ids[r], :], widened to the carrier.  `table` is [vocab, hidden] bf16, hidden % 8 == 0. */
int qwen3_embedding(const uint32_t *ids, const uint16_t *table, int rows, int hidden, int vocab, void *out, int dtype,
                    void *stream);

/* `qkv` holds, per row, q_heads query heads, then kv_heads key heads, then kv_heads value heads (128 wide each; row
 * stride `ld` elements) — the output of one projection against the concatenated Q|K|V matrix.  In place: every
 * query and key head becomes bf16(rope(bf16(rmsnorm(head, eps 1e-6) * gain))) with the rotary row of position
 * control[1] + row taken from `rope_table` ([capacity or more][128] f32: 64 cosines then 64 sines per position,
 * tools/prepare.py:90-92).  The rotated keys and the untouched values are appended to the caches at that position. */
int qwen3_prepare_qk(void *qkv, int dtype, int64_t ld, int rows, int q_heads, int kv_heads, const float *q_gain,
                     const float *k_gain, const float *rope_table, const uint32_t *control, uint16_t *k_cache, uint16_t *v_cache,
                     int capacity, void *stream);

/* out[r, h, :] = bf16(softmax(q[r, h, :] . K[0 .. control[1] + r, h / (q_heads / kv_heads), :] * 128^-0.5) . V[...]).
 * `q` may point into the qkv buffer (row stride `ldq`); `out` is [rows][q_heads * 128] with row stride `ldo`.
 * `maxima` (optional, [rows]): an atomic max of the bit patterns of |out[r, :]| is applied to maxima[r], which the
 * caller has set to the bits of 1e-8f beforehand; it feeds w8a8_quantize_with_max / W8A8_SOURCE_WITH_MAX, whose
 * result then equals that of w8a8_quantize on `out`. */
int qwen3_attention(const void *q, int dtype, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                    const uint16_t *v_cache, const uint32_t *control, void *out, int64_t ldo, int capacity, uint32_t *maxima,
                    void *stream);

/* qwen3_attention for a few rows (rows * q_heads below the SM count: decode) with the quantizer of its output folded in:
 * the CTA that finishes the last head of a row also writes the row's int8 codes ([rows][q_heads * 128]) and scale, with
 * the arithmetic of w8a8_quantize, so the O projection can follow without a quantizer launch in between (the reference
 * launches `attention` then `quantize`, src/gpu.rs:659-671 and :377-398).  Larger launches return W8A8_ERR_UNSUPPORTED. */
int qwen3_attention_quantize(const void *q, int dtype, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                             const uint16_t *v_cache, const uint32_t *control, void *out, int64_t ldo, int capacity,
                             int8_t *codes, float *scale, void *stream);

/* ---- batched decode: one new token for each of `rows` independent sequences ------------------------------------------
 * The reference serves one request at a time (GpuModel::generate, src/gpu.rs:818-929; batching is deferred,
 * docs/plans/production.md:87), so these three have no launcher of their own there: they run the arithmetic of
 * `prepare_qk` (src/kernels.rs:1350-1443) and `attention` (src/kernels.rs:1490-1658) once per row, each row against its
 * own sequence.  Row r is the newest token of sequence r: it sits at absolute position positions[r] (a device array the
 * host uploads before the step, like `control`), and sequence r's caches start `cache_stride` elements after sequence
 * r - 1's ([sequences][capacity][kv_heads][128] bf16 when dense).  A position beyond `capacity` skips the access and
 * records code 6 in the device status word. */

/* qwen3_prepare_qk for a batch of sequences: the rotary row and the cache slot of row r are those of positions[r]. */
int qwen3_prepare_qk_batched(void *qkv, int dtype, int64_t ld, int rows, int q_heads, int kv_heads, const float *q_gain,
                             const float *k_gain, const float *rope_table, const uint32_t *positions, uint16_t *k_cache,
                             uint16_t *v_cache, int capacity, int64_t cache_stride, void *stream);

/* out[r, h, :] = bf16(softmax(q[r, h, :] . K_r[0 .. positions[r], h / (q_heads / kv_heads), :] * 128^-0.5) . V_r[...]) with
 * K_r, V_r the caches of sequence r.  One CTA serves the query heads that share a key/value head, and the keys of a row
 * are split into units of 512 keys as a function of positions[r] alone, so a sequence gives the same bits whether it
 * is decoded alone or inside a batch.  The launch shape does not depend on the positions.  `workspace` (16-byte aligned, at least qwen3_attention_batched_workspace() bytes,
 * zero before the first call; the kernel leaves its counters at zero) holds the partial results of the splits; calls
 * that share a workspace must not overlap on the GPU.  `maxima` as in qwen3_attention. */
size_t qwen3_attention_batched_workspace(int rows, int q_heads, int kv_heads);
int qwen3_attention_batched(const void *q, int dtype, int64_t ldq, int rows, int q_heads, int kv_heads, const uint16_t *k_cache,
                            const uint16_t *v_cache, int64_t cache_stride, const uint32_t *positions, void *out, int64_t ldo,
                            int capacity, uint32_t *maxima, void *workspace, size_t workspace_size, void *stream);

/* `select_token` (src/kernels.rs:2191-2231; launched at src/gpu.rs:811) on stored logits [rows, n] (row stride ld):
 * token[r] = index of the largest value, the lowest index among equals, 0xffffffff if any logit of the row is not
 * finite.  `value` (optional) receives the winning logit. */
int qwen3_select_token(const void *logits, int dtype, int rows, int n, int64_t ld, uint32_t *token, float *value, void *stream);

/* The reference's own output head, `head` / `head_packed` (src/kernels.rs:2233-2373; launched at src/gpu.rs:801-809) with
 * `select_token` (src/kernels.rs:2191-2231; :811) fused in: logit[n] = bf16(sum_k x[k] * w[n, k]) for ONE row x of `hidden`
 * values (the final norm of the last position) against bf16 weights w [vocab, hidden] (bit patterns; the checkpoint keeps
 * the head unquantized, tools/prepare.py:99), the float32 sum taken in the reference's order -- lane-strided columns, then a
 * shuffle-down tree -- so the logits are bit-identical to the reference kernel's.  `logits` (optional, [vocab] in the
 * carrier `dtype`) receives them; `token` (optional) the greedy selection (largest value, lowest index among equals,
 * 0xffffffff if a logit is not finite) and `value` its logit; at least one of `logits` and `token` is required.
 * vocab <= 262144.  Calls that select a token share one per-device candidate buffer with w8a8_linear_argmax: keep them
 * in order. */
int qwen3_head_bf16(const void *x, int dtype, const uint16_t *w, int vocab, int hidden, void *logits, uint32_t *token,
                    float *value, void *stream);

/* Vocabulary split over `parts` ranks (no counterpart in the reference, which is single-GPU): candidates is
 * [parts][2][rows] = per part, `rows` tokens within the part and then the float32 bits of their logits (the `token` and
 * `value` outputs of w8a8_linear_argmax or qwen3_select_token side by side), gathered from the ranks in rank order;
 * token[r] = part * part_width + local token of the largest value (the lowest part among equals, i.e. the lowest token
 * id), or 0xffffffff if any part reported 0xffffffff or a non-finite value. */
int qwen3_merge_candidates(const uint32_t *candidates, int parts, int rows, int part_width, uint32_t *token, void *stream);

/* ---- One decode step of the whole decoder stack as a single resident kernel ------------------------------------
 * No counterpart in the reference as an interface: it runs its decode step as a captured graph of one launch per
 * operator with programmatic edges and next-weight prefetch CTAs (src/graph.rs:63-127, src/gpu.rs:318-328,
 * src/kernels.rs:173-237), which is what the launch-per-operator path of this library restates.  This entry point runs
 * the same operators, for ONE row of one sequence, inside one cooperative kernel with one CTA per SM: for every layer
 * norm_quantize -> Q|K|V projection -> prepare_qk -> attention -> quantize -> O projection + residual -> norm_quantize ->
 * gate|up projection + SwiGLU -> quantize -> down projection + residual, separated by grid-wide barriers instead of
 * kernel boundaries, each CTA quantizing the activation row for itself and requesting its share of the next matrix from
 * L2 before it waits.  The result (hidden row, KV-cache entries) is bit-identical to the separate calls
 * w8a8_rmsnorm_quantize / w8a8_linear / qwen3_prepare_qk / qwen3_attention / w8a8_quantize / w8a8_linear (residual) /
 * w8a8_linear_gate_up_swiglu / w8a8_quantize with the same inputs.
 *
 * A plan holds device copies of the layer table and the step's work buffers; creating it allocates, running it does not.
 * The weights, gains, caches and the rotary table named by the plan must stay alive and in place until it is destroyed.
 * Limits: hidden, q_heads * 128 and intermediate at most 12288 and multiples of 16; capacity <= 4096; the device must
 * support cooperative launches (W8A8_ERR_UNSUPPORTED otherwise: use the separate calls). */
struct w8a8_weight;
typedef struct qwen3_decode_plan *qwen3_decode_plan_t;
typedef struct qwen3_layer_desc {
    const void *norm1;                 /* [hidden] RMSNorm gain in front of Q|K|V, in the carrier `dtype` */
    const struct w8a8_weight *qkv;     /* [(q_heads + 2 kv_heads) * 128, hidden]: query heads, key heads, value heads */
    const float *q_gain, *k_gain;      /* [128] head-norm gains */
    const struct w8a8_weight *o;       /* [hidden, q_heads * 128] */
    const void *norm2;                 /* [hidden] RMSNorm gain in front of gate / up */
    const struct w8a8_weight *gate;    /* [intermediate, hidden] */
    const struct w8a8_weight *up;      /* [intermediate, hidden] */
    const struct w8a8_weight *down;    /* [hidden, intermediate] */
    uint16_t *k_cache, *v_cache;       /* [capacity][kv_heads][128] bf16, as for qwen3_prepare_qk */
} qwen3_layer_desc;

int qwen3_decode_plan_create(const qwen3_layer_desc *layers, int n_layers, int hidden, int q_heads, int kv_heads, int intermediate,
                             int capacity, float eps, const float *rope_table, int dtype, qwen3_decode_plan_t *plan);
int qwen3_decode_plan_destroy(qwen3_decode_plan_t plan);

/* hidden: [hidden] in the plan's carrier, the embedding row of the token on entry and the last layer's output on return.
 * control[1] is the token's position (read on the device, as in qwen3_prepare_qk); the step appends that position's key
 * and value to every layer's caches.  Queues one memset of under 1 KiB (barrier words, attention counters, row maxima)
 * and one kernel on `stream`; capturable.  Two steps of one plan must not overlap on the device.  A grid-wide wait that
 * runs out (about two seconds) ends the kernel early, leaves `hidden` undefined and code 7 in the device status word
 * (w8a8_device_status). */
int qwen3_decode_layers(qwen3_decode_plan_t plan, void *hidden, const uint32_t *control, void *stream);

/* Tensor parallel form of the step (no counterpart in the reference, which is single-GPU): the plan describes THIS rank's
 * shard (its query / key / value heads and the matching rows of Q|K|V, its slice of the input channels of O, its gate /
 * up channels and the matching input channels of down; hidden unchanged), and after this call qwen3_decode_layers runs
 * the kernel in which O and down send their partial outputs to every rank as 8-byte packets {float32 bits of the bf16
 * value, tag} with plain peer stores and every rank sums them in rank order (float32, bf16, + residual, bf16: the
 * arithmetic of w8a8_linear_allreduce).  `packet_buffers[r]` is rank r's buffer as seen from this device (symmetric /
 * peer-mapped memory, 2 * tp * hidden packets of 8 bytes, zeroed once), `seq` one local zeroed word the step advances.
 * All ranks must run the same steps in the same order; a wait for another rank's packets is bounded (about two seconds,
 * code 5 in the device status word).  tp = 1 with the rank's own buffer is valid and gives the single-GPU result. */
int qwen3_decode_plan_set_peers(qwen3_decode_plan_t plan, void *const *packet_buffers, uint32_t *seq, int rank, int tp);

/* Measurement aid: a plan created while W8A8_DECODE_TRACE=1 is in the environment makes thread 0 of every CTA note its
 * SM's cycle counter at `points` boundaries of every layer (start, after each quantizer, projection, barrier and the
 * attention step).  This call synchronises the device and copies the last step's counts to the HOST array `cycles`
 * ([ctas][layers][points] int64; counters of different CTAs are not synchronised with each other, differences within one
 * CTA are exact).  cycles == NULL only reports the three extents.  W8A8_ERR_UNSUPPORTED when the plan has no trace. */
int qwen3_decode_plan_trace(qwen3_decode_plan_t plan, int64_t *cycles, size_t capacity, int *ctas, int *layers, int *points);

/* Launches of 32 rows or more (prefill) run both attention products on the tensor cores (bf16 warp-level MMA, float32
 * accumulation, softmax weights carried as two bf16 parts); 0 keeps them on the CUDA-core kernel that shorter launches
 * use, for comparison.  Process-wide; default 1. */
int qwen3_attention_use_tensor_cores(int enabled);

#ifdef __cplusplus
}
#endif
#endif
