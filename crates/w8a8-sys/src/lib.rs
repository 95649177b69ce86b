//! Raw bindings to `libw8a8.so`, the sm_100a (B200) implementation of the W8A8 linear-layer path of
//! inferrous-qwen3: one `extern "C"` declaration per function of `include/w8a8.h` and `include/qwen3_glue.h`,
//! plus the status codes and enums of those headers.  The host keeps its own buffers, stream and graphs
//! (`crates/inferrous-qwen3/src/gpu.rs`); these calls stand where it invokes the launchers that
//! `#[cuda_module]` generates (`src/kernels.rs:322-323`).
//!
//! Pointers are device pointers unless the header says otherwise; `stream` is a `CUstream`
//! (`CudaStream::cu_stream()`); every call returns a status (`W8A8_OK` = 0) and never unwinds.
//! The documentation of each function is its comment in the C headers.
//!
//! This crate has not been compiled: the build that produced the library had no Rust toolchain.  A test of
//! the library's repository checks every declaration here against the headers (names, arity, types).
#![allow(non_camel_case_types, clippy::too_many_arguments)]

use std::os::raw::{c_char, c_int, c_void};

/// Opaque weight handle (`w8a8_weight_t`): device pointers, shape and TMA descriptors of one `[N, K]` int8 matrix.
#[repr(C)]
pub struct W8a8Weight {
    _private: [u8; 0],
}

/// Opaque plan of the resident decode kernel (`qwen3_decode_plan_t`).
#[repr(C)]
pub struct Qwen3DecodePlan {
    _private: [u8; 0],
}

/// One decoder layer as `qwen3_decode_plan_create` takes it (`qwen3_layer_desc`).
#[repr(C)]
pub struct Qwen3LayerDesc {
    pub norm1: *const c_void,
    pub qkv: *const W8a8Weight,
    pub q_gain: *const f32,
    pub k_gain: *const f32,
    pub o: *const W8a8Weight,
    pub norm2: *const c_void,
    pub gate: *const W8a8Weight,
    pub up: *const W8a8Weight,
    pub down: *const W8a8Weight,
    pub k_cache: *mut u16,
    pub v_cache: *mut u16,
}

pub const W8A8_OK: c_int = 0;
pub const W8A8_ERR_BAD_ARG: c_int = 1;
pub const W8A8_ERR_ALIGNMENT: c_int = 2;
pub const W8A8_ERR_UNSUPPORTED: c_int = 3;
pub const W8A8_ERR_CUDA: c_int = 4;
pub const W8A8_ERR_DEVICE_TIMEOUT: c_int = 5;
pub const W8A8_ERR_NOT_INITIALIZED: c_int = 6;

/// Activation carrier: 2-byte bf16 storage, or the reference's `f32` buffers holding bf16 values (`src/gpu.rs:16`).
pub const W8A8_BF16: c_int = 0;
pub const W8A8_F32: c_int = 1;

pub const W8A8_VARIANT_AUTO: c_int = 0;
pub const W8A8_VARIANT_NAIVE: c_int = 1;
pub const W8A8_VARIANT_GEMV_DP4A: c_int = 2;
pub const W8A8_VARIANT_GEMV_MMA: c_int = 3;
pub const W8A8_VARIANT_GEMM_TCGEN05: c_int = 4;
pub const W8A8_VARIANT_GEMM_SKINNY: c_int = 5;
pub const W8A8_VARIANT_GEMM_TCGEN05_PAIR: c_int = 8;
pub const W8A8_VARIANT_GEMM_CLUSTER: c_int = 9;

pub const W8A8_SOURCE_WITH_MAX: c_int = 1;
pub const W8A8_SOURCE_RMSNORM: c_int = 2;

#[link(name = "w8a8")]
extern "C" {
    // ---- include/w8a8.h: the W8A8 linear-layer path
    pub fn w8a8_init(device: c_int) -> c_int;
    pub fn w8a8_version() -> *const c_char;
    pub fn w8a8_status_string(status: c_int) -> *const c_char;
    pub fn w8a8_last_cuda_error() -> *const c_char;
    pub fn w8a8_prefetch_hint(weights: *const c_void, bytes: usize) -> c_int;
    pub fn w8a8_set_programmatic_launch(enabled: c_int) -> c_int;
    pub fn w8a8_device_status(stream: *mut c_void, detail: *mut u32) -> c_int;
    pub fn w8a8_weight_create(w: *const i8, w_scale: *const f32, n: c_int, k: c_int, out: *mut *mut W8a8Weight) -> c_int;
    pub fn w8a8_weight_destroy(weight: *mut W8a8Weight) -> c_int;
    pub fn w8a8_weight_shape(weight: *mut W8a8Weight, n: *mut c_int, k: *mut c_int) -> c_int;
    pub fn w8a8_workspace_bytes(max_rows: c_int, hidden: c_int, q_width: c_int, intermediate: c_int, offsets: *mut usize) -> usize;
    pub fn w8a8_quantize(x: *const c_void, dtype: c_int, m: c_int, k: c_int, ldx: i64, q: *mut i8, scale: *mut f32, stream: *mut c_void) -> c_int;
    pub fn w8a8_quantize_with_max(x: *const c_void, dtype: c_int, maxima: *const u32, m: c_int, k: c_int, ldx: i64, q: *mut i8, scale: *mut f32, stream: *mut c_void) -> c_int;
    pub fn w8a8_rmsnorm_quantize(x: *const c_void, gamma: *const c_void, dtype: c_int, eps: f32, m: c_int, k: c_int, ldx: i64, q: *mut i8, scale: *mut f32, y_out: *mut c_void, maxima_reset: *mut u32, stream: *mut c_void) -> c_int;
    pub fn w8a8_swiglu(gate: *const c_void, up: *const c_void, dtype: c_int, m: c_int, i: c_int, ld: i64, act: *mut c_void, maxima: *mut u32, stream: *mut c_void) -> c_int;
    pub fn w8a8_swiglu_quantize(gate: *const c_void, up: *const c_void, dtype: c_int, m: c_int, i: c_int, ld: i64, q: *mut i8, scale: *mut f32, act_out: *mut c_void, stream: *mut c_void) -> c_int;
    pub fn w8a8_residual(a: *const c_void, b: *const c_void, dtype: c_int, n: usize, out: *mut c_void, stream: *mut c_void) -> c_int;
    pub fn w8a8_linear(q: *const i8, a_scale: *const f32, weight: *mut W8a8Weight, m: c_int, residual: *const c_void, y: *mut c_void, combined: *mut c_void, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn w8a8_linear_ex(q: *const i8, a_scale: *const f32, weight: *mut W8a8Weight, m: c_int, residual: *const c_void, y: *mut c_void, combined: *mut c_void, dtype: c_int, variant: c_int, stream: *mut c_void) -> c_int;
    pub fn w8a8_linear_grouped(q: *const i8, a_scale: *const f32, weights: *const *mut W8a8Weight, count: c_int, m: c_int, outs: *const *mut c_void, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn w8a8_linear_gate_up_swiglu(q: *const i8, a_scale: *const f32, w_gate: *mut W8a8Weight, w_up: *mut W8a8Weight, m: c_int, gate_out: *mut c_void, up_out: *mut c_void, act: *mut c_void, maxima: *mut u32, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn w8a8_quantize_linear(x: *const c_void, dtype: c_int, source: c_int, gamma: *const c_void, eps: f32, maxima_in: *const u32, weight: *mut W8a8Weight, residual: *const c_void, y: *mut c_void, combined: *mut c_void, maxima_reset: *mut u32, reset_words: c_int, q_out: *mut i8, scale_out: *mut f32, stream: *mut c_void) -> c_int;
    pub fn w8a8_quantize_linear_gate_up_swiglu(x: *const c_void, dtype: c_int, source: c_int, gamma: *const c_void, eps: f32, maxima_in: *const u32, w_gate: *mut W8a8Weight, w_up: *mut W8a8Weight, act: *mut c_void, maxima_out: *mut u32, q_out: *mut i8, scale_out: *mut f32, stream: *mut c_void) -> c_int;
    pub fn w8a8_linear_no_alloc(q: *const i8, a_scale: *const f32, w: *const i8, w_scale: *const f32, m: c_int, n: c_int, k: c_int, y: *mut c_void, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn w8a8_linear_argmax(q: *const i8, a_scale: *const f32, weight: *mut W8a8Weight, m: c_int, token: *mut u32, value: *mut f32, stream: *mut c_void) -> c_int;
    pub fn w8a8_linear_allreduce(q: *const i8, a_scale: *const f32, weight: *mut W8a8Weight, m: c_int, residual: *const c_void, y: *mut c_void, combined: *mut c_void, dtype: c_int, peer_packets: *const *mut c_void, seq: *mut u32, rank: c_int, tp: c_int, slot_packets: usize, stream: *mut c_void) -> c_int;
    pub fn w8a8_tp_allreduce(partial: *const c_void, out: *mut c_void, n_el: usize, dtype: c_int, peer_bufs: *const *mut c_void, peer_flags: *const *mut u32, seq: *mut u32, rank: c_int, tp: c_int, slot_el: usize, stream: *mut c_void) -> c_int;
    pub fn w8a8_linear_acc_i32(q: *const i8, weight: *mut W8a8Weight, m: c_int, acc: *mut i32, variant: c_int, stream: *mut c_void) -> c_int;
    pub fn w8a8_rounding_probe(x: *const f32, out: *mut i8, n: usize, stream: *mut c_void) -> c_int;
    // ---- include/qwen3_glue.h: the operators around it
    pub fn qwen3_embedding(ids: *const u32, table: *const u16, rows: c_int, hidden: c_int, vocab: c_int, out: *mut c_void, dtype: c_int, stream: *mut c_void) -> c_int;
    pub fn qwen3_prepare_qk(qkv: *mut c_void, dtype: c_int, ld: i64, rows: c_int, q_heads: c_int, kv_heads: c_int, q_gain: *const f32, k_gain: *const f32, rope_table: *const f32, control: *const u32, k_cache: *mut u16, v_cache: *mut u16, capacity: c_int, stream: *mut c_void) -> c_int;
    pub fn qwen3_attention(q: *const c_void, dtype: c_int, ldq: i64, rows: c_int, q_heads: c_int, kv_heads: c_int, k_cache: *const u16, v_cache: *const u16, control: *const u32, out: *mut c_void, ldo: i64, capacity: c_int, maxima: *mut u32, stream: *mut c_void) -> c_int;
    pub fn qwen3_attention_quantize(q: *const c_void, dtype: c_int, ldq: i64, rows: c_int, q_heads: c_int, kv_heads: c_int, k_cache: *const u16, v_cache: *const u16, control: *const u32, out: *mut c_void, ldo: i64, capacity: c_int, codes: *mut i8, scale: *mut f32, stream: *mut c_void) -> c_int;
    pub fn qwen3_prepare_qk_batched(qkv: *mut c_void, dtype: c_int, ld: i64, rows: c_int, q_heads: c_int, kv_heads: c_int, q_gain: *const f32, k_gain: *const f32, rope_table: *const f32, positions: *const u32, k_cache: *mut u16, v_cache: *mut u16, capacity: c_int, cache_stride: i64, stream: *mut c_void) -> c_int;
    pub fn qwen3_attention_batched_workspace(rows: c_int, q_heads: c_int, kv_heads: c_int) -> usize;
    pub fn qwen3_attention_batched(q: *const c_void, dtype: c_int, ldq: i64, rows: c_int, q_heads: c_int, kv_heads: c_int, k_cache: *const u16, v_cache: *const u16, cache_stride: i64, positions: *const u32, out: *mut c_void, ldo: i64, capacity: c_int, maxima: *mut u32, workspace: *mut c_void, workspace_size: usize, stream: *mut c_void) -> c_int;
    pub fn qwen3_select_token(logits: *const c_void, dtype: c_int, rows: c_int, n: c_int, ld: i64, token: *mut u32, value: *mut f32, stream: *mut c_void) -> c_int;
    pub fn qwen3_head_bf16(x: *const c_void, dtype: c_int, w: *const u16, vocab: c_int, hidden: c_int, logits: *mut c_void, token: *mut u32, value: *mut f32, stream: *mut c_void) -> c_int;
    pub fn qwen3_merge_candidates(candidates: *const u32, parts: c_int, rows: c_int, part_width: c_int, token: *mut u32, stream: *mut c_void) -> c_int;
    pub fn qwen3_decode_plan_create(layers: *const Qwen3LayerDesc, n_layers: c_int, hidden: c_int, q_heads: c_int, kv_heads: c_int, intermediate: c_int, capacity: c_int, eps: f32, rope_table: *const f32, dtype: c_int, plan: *mut *mut Qwen3DecodePlan) -> c_int;
    pub fn qwen3_decode_plan_destroy(plan: *mut Qwen3DecodePlan) -> c_int;
    pub fn qwen3_decode_layers(plan: *mut Qwen3DecodePlan, hidden: *mut c_void, control: *const u32, stream: *mut c_void) -> c_int;
    pub fn qwen3_decode_plan_set_peers(plan: *mut Qwen3DecodePlan, packet_buffers: *const *mut c_void, seq: *mut u32, rank: c_int, tp: c_int) -> c_int;
    pub fn qwen3_decode_plan_trace(plan: *mut Qwen3DecodePlan, cycles: *mut i64, capacity: usize, ctas: *mut c_int, layers: *mut c_int, points: *mut c_int) -> c_int;
    pub fn qwen3_attention_use_tensor_cores(enabled: c_int) -> c_int;
}

/// `Err(status)` unless the call returned `W8A8_OK`; the text of a failing CUDA call is in `w8a8_last_cuda_error()`.
pub fn check(status: c_int) -> Result<(), c_int> {
    if status == W8A8_OK {
        Ok(())
    } else {
        Err(status)
    }
}
