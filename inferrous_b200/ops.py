"""Host-side mirror of the reference host runtime's W8A8 operator methods, over the C ABI.

Names and argument meaning follow `GpuModel` in crates/inferrous-qwen3/src/gpu.rs:
`norm_quantize` (:340), `linear_residual` (:364), `quantize` (:424), `linear_quantized`
(:450), `residual` (:510), and the direct launches of `linear_triple` (:571-590),
`linear_swiglu` (:730-745) and `swiglu` (:770-777); `Matrix` is gpu::Matrix (:43-49).
Like the reference's methods, every call takes caller-owned OUTPUT buffers and queues work
on one stream; nothing here allocates, synchronises or falls back to the CPU.

torch supplies device memory and the stream.  Activation tensors are torch.bfloat16
(2-byte storage) or torch.float32 (the reference's carrier for bf16-valued activations).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi

_initialised: set[int] = set()


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return capi.BF16
    if t.dtype == torch.float32:
        return capi.F32
    raise TypeError(f"activation dtype must be bfloat16 or float32, got {t.dtype}")


def _ptr(t: torch.Tensor | None):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("w8a8 ops take CUDA tensors only (there is no CPU path)")
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def init(device: int | None = None) -> None:
    """`device::load(&ctx)` (src/gpu.rs:250): load kernels for a device, once, before capture."""
    if not torch.cuda.is_available():
        raise RuntimeError("inferrous_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
    dev = torch.cuda.current_device() if device is None else device
    if dev not in _initialised:
        capi.check(capi.load().w8a8_init(dev), "w8a8_init")
        _initialised.add(dev)


def set_programmatic_launch(enabled: bool) -> None:
    """The reference's CLEAN_PDL switch (src/gpu.rs:317): launch every hot-path kernel with a programmatic edge."""
    capi.check(capi.load().w8a8_set_programmatic_launch(1 if enabled else 0), "w8a8_set_programmatic_launch")


def prefetch_hint(weights: torch.Tensor | None, offset_bytes: int = 0, nbytes: int | None = None) -> None:
    """Attach an L2 prefetch of (part of) an immutable weight tensor to the next attention launch of this thread
    (the reference's next-weight prefetch, src/gpu.rs:19-42)."""
    if weights is None:
        capi.check(capi.load().w8a8_prefetch_hint(None, 0), "w8a8_prefetch_hint")
        return
    total = weights.numel() * weights.element_size()
    nbytes = total - offset_bytes if nbytes is None else min(nbytes, total - offset_bytes)
    if nbytes <= 0:
        return
    capi.check(capi.load().w8a8_prefetch_hint(C.c_void_p(weights.data_ptr() + offset_bytes), nbytes), "w8a8_prefetch_hint")


def device_status() -> tuple[int, int]:
    """(status, detail) of the device-side bounded waits; synchronises the current stream."""
    detail = C.c_uint32(0)
    st = capi.load().w8a8_device_status(_stream(), C.byref(detail))
    return st, detail.value


class Matrix:
    """gpu::Matrix {w, map, scale, k, n} (src/gpu.rs:43-49): an immutable int8 weight [N,K] with
    one f32 scale per output channel.  The TMA descriptor lives inside the C handle."""

    def __init__(self, w: torch.Tensor, scale: torch.Tensor):
        assert w.dtype == torch.int8 and w.dim() == 2 and w.is_contiguous() and w.is_cuda
        assert scale.dtype == torch.float32 and scale.numel() == w.shape[0] and scale.is_contiguous()
        init(w.device.index)
        self.w, self.scale = w, scale
        self.n, self.k = w.shape
        h = C.c_void_p()
        capi.check(capi.load().w8a8_weight_create(_ptr(w), _ptr(scale), self.n, self.k, C.byref(h)), "w8a8_weight_create")
        self.handle = h

    def __del__(self):
        h = getattr(self, "handle", None)
        if h and capi is not None:  # module globals are already cleared when the interpreter shuts down
            capi.load().w8a8_weight_destroy(h)
            self.handle = None


class Workspace:
    """The hot path's share of gpu::Workspace (src/gpu.rs:76-143): int8 scratch for the two
    activation widths, per-row scales and SwiGLU maxima."""

    def __init__(self, rows: int, device, hidden: int = 4096, intermediate: int = 12288):
        self.quant4 = torch.empty((rows, hidden), dtype=torch.int8, device=device)
        self.quant12 = torch.empty((rows, intermediate), dtype=torch.int8, device=device)
        self.scales = torch.empty((rows,), dtype=torch.float32, device=device)
        self.maxima = torch.full((rows,), 0x322BCC77, dtype=torch.int32, device=device)  # 1e-8f bits


def quantize(x: torch.Tensor, q: torch.Tensor, scale: torch.Tensor) -> None:
    """GpuModel::quantize (src/gpu.rs:424-449) -> kernel `quantize` (src/kernels.rs:415-452)."""
    M, K = x.shape
    capi.check(capi.load().w8a8_quantize(_ptr(x), _dtype_code(x), M, K, x.stride(0), _ptr(q), _ptr(scale), _stream()),
               "w8a8_quantize")


def quantize_with_max(x: torch.Tensor, maxima: torch.Tensor, q: torch.Tensor, scale: torch.Tensor) -> None:
    """Kernel `quantize_with_max` (src/kernels.rs:455-475; src/gpu.rs:377-390)."""
    M, K = x.shape
    capi.check(capi.load().w8a8_quantize_with_max(_ptr(x), _dtype_code(x), _ptr(maxima), M, K, x.stride(0), _ptr(q),
                                                  _ptr(scale), _stream()), "w8a8_quantize_with_max")


def norm_quantize(x: torch.Tensor, gain: torch.Tensor, out: torch.Tensor | None, q: torch.Tensor, scale: torch.Tensor,
                  maxima: torch.Tensor | None, eps: float = 1e-6) -> None:
    """GpuModel::norm_quantize (src/gpu.rs:340-363) -> kernel `norm_quantize` (src/kernels.rs:479-576).
    `out` (the bf16 norm row, only ever read by tracing in the reference) may be None."""
    M, K = x.shape
    assert gain.dtype == x.dtype
    capi.check(capi.load().w8a8_rmsnorm_quantize(_ptr(x), _ptr(gain), _dtype_code(x), eps, M, K, x.stride(0), _ptr(q),
                                                 _ptr(scale), _ptr(out), _ptr(maxima), _stream()), "w8a8_rmsnorm_quantize")


def swiglu(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor, maxima: torch.Tensor | None) -> None:
    """Kernel `swiglu` (src/kernels.rs:2172-2190; src/gpu.rs:770-777)."""
    M, I = gate.shape
    assert gate.stride(0) == up.stride(0)
    capi.check(capi.load().w8a8_swiglu(_ptr(gate), _ptr(up), _dtype_code(gate), M, I, gate.stride(0), _ptr(out),
                                       _ptr(maxima), _stream()), "w8a8_swiglu")


def swiglu_quantize(gate: torch.Tensor, up: torch.Tensor, q: torch.Tensor, scale: torch.Tensor,
                    act: torch.Tensor | None = None) -> None:
    """`swiglu` + `quantize` of the down-projection input in one pass (src/gpu.rs:768-778 + :377-398)."""
    M, I = gate.shape
    assert gate.stride(0) == up.stride(0)
    capi.check(capi.load().w8a8_swiglu_quantize(_ptr(gate), _ptr(up), _dtype_code(gate), M, I, gate.stride(0), _ptr(q),
                                                _ptr(scale), _ptr(act), _stream()), "w8a8_swiglu_quantize")


def residual(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """GpuModel::residual (src/gpu.rs:510-517) -> kernel `residual` (src/kernels.rs:2163-2170)."""
    capi.check(capi.load().w8a8_residual(_ptr(a), _ptr(b), _dtype_code(a), a.numel(), _ptr(out), _stream()), "w8a8_residual")


def linear_quantized(q: torch.Tensor, scale: torch.Tensor, w: Matrix, out: torch.Tensor,
                     variant: int = capi.VARIANT_AUTO) -> None:
    """GpuModel::linear_quantized (src/gpu.rs:450-509): regime chosen from the row count."""
    M = q.shape[0]
    capi.check(capi.load().w8a8_linear_ex(_ptr(q), _ptr(scale), w.handle, M, None, _ptr(out), None, _dtype_code(out),
                                          variant, _stream()), "w8a8_linear")


def linear_residual(q: torch.Tensor, scale: torch.Tensor, w: Matrix, out: torch.Tensor | None, residual_in: torch.Tensor,
                    combined: torch.Tensor, variant: int = capi.VARIANT_AUTO) -> None:
    """The projection half of GpuModel::linear_residual (src/gpu.rs:400-421): kernel `linear_residual`
    (src/kernels.rs:579-618) in decode, `linear_*` + `residual` in prefill.  `out` may be None."""
    M = q.shape[0]
    capi.check(capi.load().w8a8_linear_ex(_ptr(q), _ptr(scale), w.handle, M, _ptr(residual_in), _ptr(out), _ptr(combined),
                                          _dtype_code(combined), variant, _stream()), "w8a8_linear(residual)")


def linear_grouped(q: torch.Tensor, scale: torch.Tensor, ws: list[Matrix], outs: list[torch.Tensor]) -> None:
    """Kernels `linear_pair` / `linear_triple` (src/kernels.rs:698-806; src/gpu.rs:571-590)."""
    n = len(ws)
    handles = (C.c_void_p * n)(*[w.handle for w in ws])
    optrs = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
    capi.check(capi.load().w8a8_linear_grouped(_ptr(q), _ptr(scale), handles, n, q.shape[0], optrs, _dtype_code(outs[0]),
                                               _stream()), "w8a8_linear_grouped")


def linear_swiglu(q: torch.Tensor, scale: torch.Tensor, w_gate: Matrix, w_up: Matrix, gate: torch.Tensor | None,
                  up: torch.Tensor | None, act: torch.Tensor, maxima: torch.Tensor | None) -> None:
    """Kernel `linear_swiglu` (src/kernels.rs:621-695; src/gpu.rs:730-745)."""
    capi.check(capi.load().w8a8_linear_gate_up_swiglu(_ptr(q), _ptr(scale), w_gate.handle, w_up.handle, q.shape[0],
                                                      _ptr(gate), _ptr(up), _ptr(act), _ptr(maxima), _dtype_code(act),
                                                      _stream()), "w8a8_linear_gate_up_swiglu")


def quantize_linear(x: torch.Tensor, w: Matrix, out: torch.Tensor | None, *, gain: torch.Tensor | None = None,
                    maxima_in: torch.Tensor | None = None, eps: float = 1e-6, residual_in: torch.Tensor | None = None,
                    combined: torch.Tensor | None = None, maxima_reset: torch.Tensor | None = None,
                    q_out: torch.Tensor | None = None, scale_out: torch.Tensor | None = None) -> None:
    """One token: `norm_quantize` (gain given) or `quantize_with_max` (maxima_in given) folded into the projection that
    follows it (GpuModel::norm_quantize / linear_residual at one row, src/gpu.rs:340-423)."""
    source = capi.SOURCE_RMSNORM if gain is not None else capi.SOURCE_WITH_MAX
    capi.check(capi.load().w8a8_quantize_linear(_ptr(x), _dtype_code(x), source, _ptr(gain), eps, _ptr(maxima_in), w.handle,
                                                _ptr(residual_in), _ptr(out), _ptr(combined), _ptr(maxima_reset),
                                                0 if maxima_reset is None else maxima_reset.numel(), _ptr(q_out),
                                                _ptr(scale_out), _stream()), "w8a8_quantize_linear")


def quantize_linear_swiglu(x: torch.Tensor, w_gate: Matrix, w_up: Matrix, act: torch.Tensor, maxima_out: torch.Tensor | None, *,
                           gain: torch.Tensor | None = None, maxima_in: torch.Tensor | None = None, eps: float = 1e-6,
                           q_out: torch.Tensor | None = None, scale_out: torch.Tensor | None = None) -> None:
    """One token: the quantizer folded into kernel `linear_swiglu` (src/kernels.rs:621-695; src/gpu.rs:730-745)."""
    source = capi.SOURCE_RMSNORM if gain is not None else capi.SOURCE_WITH_MAX
    capi.check(capi.load().w8a8_quantize_linear_gate_up_swiglu(_ptr(x), _dtype_code(x), source, _ptr(gain), eps, _ptr(maxima_in),
                                                               w_gate.handle, w_up.handle, _ptr(act), _ptr(maxima_out),
                                                               _ptr(q_out), _ptr(scale_out), _stream()),
               "w8a8_quantize_linear_gate_up_swiglu")


def linear_no_alloc(q: torch.Tensor, scale: torch.Tensor, w: torch.Tensor, w_scale: torch.Tensor, out: torch.Tensor) -> None:
    """The projection for callers that cannot allocate device memory (w8a8_linear_no_alloc): raw weight
    tensors instead of a Matrix handle, at most 16 tokens, scratch in a fixed array inside the library.
    Needs no init(); calls on different streams must not overlap."""
    N, K = w.shape
    capi.check(capi.load().w8a8_linear_no_alloc(_ptr(q), _ptr(scale), _ptr(w), _ptr(w_scale), q.shape[0], N, K, _ptr(out),
                                                _dtype_code(out), _stream()), "w8a8_linear_no_alloc")


def linear_argmax(q: torch.Tensor, scale: torch.Tensor, w: Matrix, token: torch.Tensor, value: torch.Tensor | None = None) -> None:
    """Head projection + `select_token` (src/kernels.rs:2191-2231) in one pass: token[m] = index of the largest logit
    (lowest index among equals, 0xffffffff if any logit is not finite); the logits are never written."""
    capi.check(capi.load().w8a8_linear_argmax(_ptr(q), _ptr(scale), w.handle, q.shape[0], _ptr(token), _ptr(value), _stream()),
               "w8a8_linear_argmax")


def linear_acc_i32(q: torch.Tensor, w: Matrix, acc: torch.Tensor, variant: int = capi.VARIANT_NAIVE) -> None:
    """Raw int32 accumulators (parity checks against the CPU-integer fixtures)."""
    capi.check(capi.load().w8a8_linear_acc_i32(_ptr(q), w.handle, q.shape[0], _ptr(acc), variant, _stream()),
               "w8a8_linear_acc_i32")


def rounding_probe(x: torch.Tensor, out: torch.Tensor) -> None:
    """Kernel `rounding_probe` (src/kernels.rs:326-333)."""
    capi.check(capi.load().w8a8_rounding_probe(_ptr(x), _ptr(out), x.numel(), _stream()), "w8a8_rounding_probe")


# ---- the operators around the linear layers (include/qwen3_glue.h) ---------------------------------------

def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """Kernel `embedding` (src/kernels.rs:335-345; src/gpu.rs:543-551): out[r] = table[ids[r]].  `ids` is uint32
    (or int32 holding non-negative ids) on the device; in decode it is the control buffer, whose word 0 is the token."""
    rows, hidden = out.shape
    capi.check(capi.load().qwen3_embedding(_ptr(ids), _ptr(table), rows, hidden, table.shape[0], _ptr(out), _dtype_code(out),
                                           _stream()), "qwen3_embedding")


def prepare_qk(qkv: torch.Tensor, q_heads: int, kv_heads: int, q_gain: torch.Tensor, k_gain: torch.Tensor,
               rope_table: torch.Tensor, control: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    """Kernel `prepare_qk` (src/kernels.rs:1350-1443; src/gpu.rs:626-641): in-place head RMSNorm + RoPE of the query
    and key heads of `qkv` ([rows, (q_heads + 2 kv_heads) * 128]) and append of keys / values to the caches
    ([capacity, kv_heads, 128] bf16) at position control[1] + row."""
    capi.check(capi.load().qwen3_prepare_qk(_ptr(qkv), _dtype_code(qkv), qkv.stride(0), qkv.shape[0], q_heads, kv_heads,
                                            _ptr(q_gain), _ptr(k_gain), _ptr(rope_table), _ptr(control), _ptr(k_cache),
                                            _ptr(v_cache), k_cache.shape[0], _stream()), "qwen3_prepare_qk")


def attention(q: torch.Tensor, q_heads: int, kv_heads: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
              control: torch.Tensor, out: torch.Tensor, maxima: torch.Tensor | None = None) -> None:
    """Kernel `attention` (src/kernels.rs:1490-1658; src/gpu.rs:659-671): causal grouped-query attention of `rows`
    new positions over the cache.  `q` may be the qkv buffer (its leading q_heads * 128 columns are read).  `maxima`
    ([rows] words preset to the bits of 1e-8f) receives max |out| per row for quantize_with_max."""
    capi.check(capi.load().qwen3_attention(_ptr(q), _dtype_code(q), q.stride(0), q.shape[0], q_heads, kv_heads, _ptr(k_cache),
                                           _ptr(v_cache), _ptr(control), _ptr(out), out.stride(0), k_cache.shape[0], _ptr(maxima),
                                           _stream()), "qwen3_attention")


def attention_use_tensor_cores(enabled: bool) -> None:
    """Many-row attention launches on the tensor cores (default) or on the CUDA-core kernel (comparison runs)."""
    capi.check(capi.load().qwen3_attention_use_tensor_cores(1 if enabled else 0), "qwen3_attention_use_tensor_cores")


def attention_quantize(q: torch.Tensor, q_heads: int, kv_heads: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                       control: torch.Tensor, out: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor) -> None:
    """`attention` for a few rows with `quantize` of its output folded in (decode): the O projection's input codes and
    scale come out of the attention launch itself."""
    capi.check(capi.load().qwen3_attention_quantize(_ptr(q), _dtype_code(q), q.stride(0), q.shape[0], q_heads, kv_heads,
                                                    _ptr(k_cache), _ptr(v_cache), _ptr(control), _ptr(out), out.stride(0),
                                                    k_cache.shape[0], _ptr(codes), _ptr(scale), _stream()),
               "qwen3_attention_quantize")


# ---- batched decode: one new token for each of `rows` independent sequences --------------------------------

def prepare_qk_batched(qkv: torch.Tensor, q_heads: int, kv_heads: int, q_gain: torch.Tensor, k_gain: torch.Tensor,
                       rope_table: torch.Tensor, positions: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    """`prepare_qk` (src/kernels.rs:1350-1443) per sequence: row r of `qkv` is the newest token of sequence r, at
    position positions[r]; the caches are [sequences, capacity, kv_heads, 128] bf16."""
    assert k_cache.dim() == 4 and k_cache.shape[0] >= qkv.shape[0] and k_cache.stride() == v_cache.stride()
    capi.check(capi.load().qwen3_prepare_qk_batched(_ptr(qkv), _dtype_code(qkv), qkv.stride(0), qkv.shape[0], q_heads, kv_heads,
                                                    _ptr(q_gain), _ptr(k_gain), _ptr(rope_table), _ptr(positions), _ptr(k_cache),
                                                    _ptr(v_cache), k_cache.shape[1], k_cache.stride(0), _stream()),
               "qwen3_prepare_qk_batched")


def attention_batched_workspace(rows: int, q_heads: int, kv_heads: int, device="cuda") -> torch.Tensor:
    """Zeroed scratch for attention_batched (partial results of the key splits and their arrival counters)."""
    nbytes = capi.load().qwen3_attention_batched_workspace(rows, q_heads, kv_heads)
    return torch.zeros((nbytes + 3) // 4, dtype=torch.int32, device=device)


def attention_batched(q: torch.Tensor, q_heads: int, kv_heads: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      positions: torch.Tensor, out: torch.Tensor, workspace: torch.Tensor, maxima: torch.Tensor | None = None) -> None:
    """`attention` (src/kernels.rs:1490-1658) per sequence: row r attends to keys 0 .. positions[r] of sequence r's cache."""
    assert k_cache.dim() == 4 and k_cache.shape[0] >= q.shape[0] and k_cache.stride() == v_cache.stride()
    capi.check(capi.load().qwen3_attention_batched(_ptr(q), _dtype_code(q), q.stride(0), q.shape[0], q_heads, kv_heads, _ptr(k_cache),
                                                   _ptr(v_cache), k_cache.stride(0), _ptr(positions), _ptr(out), out.stride(0),
                                                   k_cache.shape[1], _ptr(maxima), _ptr(workspace),
                                                   workspace.numel() * workspace.element_size(), _stream()), "qwen3_attention_batched")


def select_token(logits: torch.Tensor, token: torch.Tensor, value: torch.Tensor | None = None) -> None:
    """Kernel `select_token` (src/kernels.rs:2191-2231; src/gpu.rs:811) per row of stored logits."""
    rows, n = logits.shape
    capi.check(capi.load().qwen3_select_token(_ptr(logits), _dtype_code(logits), rows, n, logits.stride(0), _ptr(token), _ptr(value),
                                              _stream()), "qwen3_select_token")


def merge_candidates(candidates: torch.Tensor, part_width: int, token: torch.Tensor) -> None:
    """Vocabulary-split head: candidates [parts, 2, rows] = per part the tokens within the part, then the bits of their
    logits -> global token per row."""
    parts, _, rows = candidates.shape
    capi.check(capi.load().qwen3_merge_candidates(_ptr(candidates), parts, rows, part_width, _ptr(token), _stream()),
               "qwen3_merge_candidates")


def head_bf16(x: torch.Tensor, w: torch.Tensor, logits: torch.Tensor | None = None, token: torch.Tensor | None = None,
              value: torch.Tensor | None = None) -> None:
    """Kernels `head` / `head_packed` + `select_token` (src/kernels.rs:2233-2373, :2191-2231; src/gpu.rs:801-811): the
    reference's bf16 head on one row `x` ([1, hidden] or [hidden]) against `w` ([vocab, hidden] torch.bfloat16), logits
    bit-identical to the reference's summation order; `token` receives the greedy selection."""
    vocab, hidden = w.shape
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and x.numel() == hidden
    capi.check(capi.load().qwen3_head_bf16(_ptr(x), _dtype_code(x), _ptr(w), vocab, hidden, _ptr(logits), _ptr(token), _ptr(value),
                                           _stream()), "qwen3_head_bf16")


class DecodePlan:
    """qwen3_decode_plan (include/qwen3_glue.h): one decode step of the whole decoder stack as a single resident kernel.
    `layers` is a sequence of objects with norm1, qkv, qnorm, knorm, o, norm2, gate, up, down (Matrix handles and gain
    tensors); k_caches / v_caches the per-layer [capacity, kv_heads, 128] bf16 caches.  The plan keeps references to
    everything it names.  Raises W8A8Error (status 3) where the shape or the device is not supported."""

    def __init__(self, layers, k_caches, v_caches, hidden: int, q_heads: int, kv_heads: int, intermediate: int, eps: float,
                 rope: torch.Tensor, dtype: torch.dtype = torch.bfloat16):
        init(rope.device.index)
        assert rope.dtype == torch.float32 and rope.is_contiguous() and rope.shape[1] == 128
        self._keep = (list(layers), list(k_caches), list(v_caches), rope)
        table = (capi.LayerDesc * len(layers))()
        for d, layer, k, v in zip(table, layers, k_caches, v_caches):
            assert layer.norm1.dtype == dtype and layer.norm2.dtype == dtype and layer.qnorm.dtype == torch.float32
            assert k.is_contiguous() and v.is_contiguous() and k.shape == v.shape and tuple(k.shape[1:]) == (kv_heads, 128)
            d.norm1, d.norm2, d.q_gain, d.k_gain = (_ptr(t).value for t in (layer.norm1, layer.norm2, layer.qnorm, layer.knorm))
            d.qkv, d.o, d.gate, d.up, d.down = (m.handle.value for m in (layer.qkv, layer.o, layer.gate, layer.up, layer.down))
            d.k_cache, d.v_cache = _ptr(k).value, _ptr(v).value
        capacity = k_caches[0].shape[0]
        handle = C.c_void_p()
        capi.check(capi.load().qwen3_decode_plan_create(C.cast(table, C.c_void_p), len(layers), hidden, q_heads, kv_heads, intermediate,
                                                        capacity, eps, _ptr(rope), 0 if dtype == torch.bfloat16 else 1,
                                                        C.byref(handle)), "qwen3_decode_plan_create")
        self.handle = handle
        self.hidden = hidden

    def set_peers(self, packet_buffers, seq: torch.Tensor, rank: int, tp: int) -> None:
        """Tensor parallel (qwen3_decode_plan_set_peers): `packet_buffers` are the device addresses of every rank's packet
        buffer (2 * tp * hidden packets of 8 bytes, zeroed), `seq` a zeroed int32 word of this rank."""
        table = (C.c_void_p * tp)(*[int(p) for p in packet_buffers])
        self._keep = self._keep + (seq,)
        capi.check(capi.load().qwen3_decode_plan_set_peers(self.handle, table, _ptr(seq), rank, tp), "qwen3_decode_plan_set_peers")

    def run(self, hidden_row: torch.Tensor, control: torch.Tensor) -> None:
        """hidden_row ([hidden] or [1, hidden]): the token's embedding in, the last layer's output out; control = {token,
        position} on the device."""
        assert hidden_row.numel() == self.hidden and hidden_row.is_contiguous()
        capi.check(capi.load().qwen3_decode_layers(self.handle, _ptr(hidden_row), _ptr(control), _stream()), "qwen3_decode_layers")

    def __del__(self):
        h = getattr(self, "handle", None)
        if h and capi is not None:
            capi.load().qwen3_decode_plan_destroy(h)
            self.handle = None

    def trace(self):
        """Cycle counts of the last step, [ctas, layers, points] (numpy int64), when the plan was created with
        W8A8_DECODE_TRACE=1 in the environment (qwen3_decode_plan_trace)."""
        import numpy as np

        ctas, layers, points = C.c_int(), C.c_int(), C.c_int()
        lib = capi.load()
        capi.check(lib.qwen3_decode_plan_trace(self.handle, None, 0, C.byref(ctas), C.byref(layers), C.byref(points)),
                   "qwen3_decode_plan_trace")
        out = np.zeros((ctas.value, layers.value, points.value), dtype=np.int64)
        capi.check(lib.qwen3_decode_plan_trace(self.handle, out.ctypes.data_as(C.c_void_p), out.size, C.byref(ctas), C.byref(layers),
                                               C.byref(points)), "qwen3_decode_plan_trace")
        return out
