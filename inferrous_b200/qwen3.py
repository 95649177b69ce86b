"""A Qwen3 W8A8 forward pass and greedy generation loop over the C ABI: the caller of the linear-layer path.

Mirrors `GpuModel::forward` and `GpuModel::generate` of the reference host
(crates/inferrous-qwen3/src/gpu.rs:528-817 and :818-929): embedding, then per layer
norm_quantize -> Q|K|V projection -> prepare_qk -> attention -> quantize -> O projection + residual ->
norm_quantize -> gate/up projection + SwiGLU -> quantize -> down projection + residual, then the final norm,
the head projection and greedy selection.  Every device operation is a kernel of libw8a8.so; torch supplies
memory, the stream and CUDA-graph capture only.  As in the reference, prefill runs eagerly, one decode step is
captured once and replayed (src/gpu.rs:303-333), and the host writes {token, position} into the control buffer
and reads the selected token back every step (src/gpu.rs:876-906).

Differences from the reference host, all outside the linear-layer arithmetic:
  * Q, K and V (and gate, up) are stored as one concatenated matrix each; with per-output-channel scales the
    concatenated projection equals the separate ones channel for channel.
  * Two output heads: the reference's bf16 head (Qwen3Weights.head_bf16; what a loaded bundle uses, logits bit-identical
    to the reference's `head` kernel, src/gpu.rs:801-809) and a W8A8 head like the body (the benchmark's lm_head shape;
    the final norm is then fused with a quantizer).  Either way the greedy selection is fused into the head kernel.
  * Activations are stored as bf16 (the reference stores the same values in f32 buffers).
"""
from __future__ import annotations

import dataclasses
import math
import os

import torch

from . import capi, ops


@dataclasses.dataclass(frozen=True)
class Qwen3Config:
    layers: int = 36
    hidden: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    intermediate: int = 12288
    vocab: int = 151936
    context: int = 4096
    rope_theta: float = 1e6
    eps: float = 1e-6
    head_dim: int = 128  # fixed by the kernels

    @property
    def q_width(self) -> int:
        return self.q_heads * self.head_dim

    @property
    def qkv_width(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim

    @classmethod
    def qwen3_8b(cls) -> "Qwen3Config":
        return cls()

    def weight_bytes(self) -> int:
        """int8 bytes one decode step streams (body + head), the numerator of the bandwidth figure."""
        per_layer = self.hidden * self.qkv_width + self.q_width * self.hidden + 3 * self.hidden * self.intermediate
        return self.layers * per_layer + self.vocab * self.hidden


def rope_table(config: Qwen3Config) -> torch.Tensor:
    """[context, 128] float32: 64 cosines then 64 sines per position, computed as the reference's bundle
    preparation does (tools/prepare.py:90-92), on the CPU."""
    freq = 1.0 / (config.rope_theta ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
    angles = torch.arange(config.context, dtype=torch.float32)[:, None] * freq
    return torch.cat([angles.cos(), angles.sin()], dim=1)


class Layer:
    """One decoder layer's tensors: gains in the activation dtype (head gains float32) and gpu::Matrix handles."""

    def __init__(self, config: Qwen3Config, norm1, qkv, qkv_scale, qnorm, knorm, o, o_scale, norm2, gate_up, gate_up_scale,
                 down, down_scale):
        inter = config.intermediate
        self.norm1, self.norm2 = norm1, norm2
        self.qnorm, self.knorm = qnorm, knorm
        self.qkv = ops.Matrix(qkv, qkv_scale)
        self.o = ops.Matrix(o, o_scale)
        self.gate_up = ops.Matrix(gate_up, gate_up_scale)            # prefill: one projection, then swiglu_quantize
        self.gate = ops.Matrix(gate_up[:inter], gate_up_scale[:inter])  # decode: fused gate/up + SwiGLU kernel
        self.up = ops.Matrix(gate_up[inter:], gate_up_scale[inter:])
        self.down = ops.Matrix(down, down_scale)


class Qwen3Weights:
    def __init__(self, config: Qwen3Config, embedding, layers, final_gain, head, head_scale, device, head_bf16=None):
        """`head`, `head_scale`: the W8A8 output head (int8 [vocab, hidden] + channel scales).  `head_bf16` ([vocab, hidden]
        torch.bfloat16): the reference's own unquantized head (src/gpu.rs:801-809); when given, generation uses it
        (ops.head_bf16, logits bit-identical to the reference's kernel) and the W8A8 head may be None."""
        self.config = config
        self.embedding = embedding
        self.layers = layers
        self.final_gain = final_gain
        self.head = ops.Matrix(head, head_scale) if head is not None else None
        self.head_bf16 = head_bf16
        if self.head is None and head_bf16 is None:
            raise ValueError("a model needs an output head")
        self.rope = rope_table(config).to(device)
        self.tp, self.rank = 1, 0          # tensor-parallel degree and this process's rank (see shard())
        self.full_config = config          # the unsharded model

    def shard(self, rank: int, tp: int) -> "Qwen3Weights":
        """This rank's share of the model under tensor parallelism (inferrous_b200/tp.py): query / key / value heads and
        gate / up channels by output rows, O and down by input columns (their partial outputs are summed by an
        all-reduce), the head by vocabulary rows; embedding, gains and the rotary table are replicated."""
        from . import tp as tpmod

        if tp == 1:
            return self
        c = self.config
        if c.vocab % tp:
            raise ValueError(f"vocabulary {c.vocab} cannot be split {tp} ways")
        local = dataclasses.replace(c, q_heads=c.q_heads // tp, kv_heads=c.kv_heads // tp, intermediate=c.intermediate // tp)
        qw, il = local.q_width, local.intermediate
        layers = []
        for l in self.layers:
            qkv, qkv_s = tpmod.take_rows(l.qkv.w, l.qkv.scale, tpmod.qkv_rows(c.q_heads, c.kv_heads, rank, tp))
            gu, gu_s = tpmod.take_rows(l.gate_up.w, l.gate_up.scale, tpmod.gate_up_rows(c.intermediate, rank, tp))
            o = l.o.w[:, rank * qw:(rank + 1) * qw].contiguous()
            down = l.down.w[:, rank * il:(rank + 1) * il].contiguous()
            layers.append(Layer(local, l.norm1, qkv, qkv_s, l.qnorm, l.knorm, o, l.o.scale, l.norm2, gu, gu_s, down, l.down.scale))
        vl = c.vocab // tp
        rows = slice(rank * vl, (rank + 1) * vl)
        out = Qwen3Weights(local, self.embedding, layers, self.final_gain,
                           self.head.w[rows].contiguous() if self.head is not None else None,
                           self.head.scale[rows].contiguous() if self.head is not None else None, self.embedding.device,
                           head_bf16=self.head_bf16[rows].contiguous() if self.head_bf16 is not None else None)
        out.rope = self.rope
        out.tp, out.rank, out.full_config = tp, rank, c
        return out

    @classmethod
    def random(cls, config: Qwen3Config, seed: int = 0, device="cuda") -> "Qwen3Weights":
        """Random-init weights of the architecture: uniform int8 codes, channel scales sized so that every
        projection keeps the activation variance (the codes of a row quantized to +-127 have a standard deviation
        near 30, uniform weight codes near 73)."""
        ops.init()
        gen = torch.Generator(device=device).manual_seed(seed)
        act = torch.bfloat16

        def matrix(n, k):
            w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=device, generator=gen)
            s = (0.5 + torch.rand(n, device=device, generator=gen)) / (69.0 * math.sqrt(k))
            return w, s.float()

        def gain(n, dtype):
            return (1.0 + 0.1 * torch.randn(n, device=device, generator=gen)).to(dtype)

        layers = []
        for _ in range(config.layers):
            qkv, qkv_s = matrix(config.qkv_width, config.hidden)
            o, o_s = matrix(config.hidden, config.q_width)
            gu, gu_s = matrix(2 * config.intermediate, config.hidden)
            down, down_s = matrix(config.hidden, config.intermediate)
            layers.append(Layer(config, gain(config.hidden, act), qkv, qkv_s, gain(128, torch.float32), gain(128, torch.float32),
                                o, o_s, gain(config.hidden, act), gu, gu_s, down, down_s))
        embedding = torch.randn(config.vocab, config.hidden, device=device, generator=gen).to(act)
        head, head_s = matrix(config.vocab, config.hidden)
        return cls(config, embedding, layers, gain(config.hidden, act), head, head_s, device)


class Workspace:
    """gpu::Workspace (src/gpu.rs:76-143) for a fixed row count."""

    def __init__(self, config: Qwen3Config, rows: int, device="cuda", wide_gate_up: bool = True):
        act = torch.bfloat16
        self.rows = rows
        self.hidden = torch.empty(rows, config.hidden, dtype=act, device=device)
        self.residual = torch.empty(rows, config.hidden, dtype=act, device=device)
        self.qkv = torch.empty(rows, config.qkv_width, dtype=act, device=device)
        self.attention = torch.empty(rows, config.q_width, dtype=act, device=device)
        self.gate_up = torch.empty(rows, 2 * config.intermediate, dtype=act, device=device) if wide_gate_up else None
        self.act = torch.empty(rows, config.intermediate, dtype=act, device=device)
        self.quant4 = torch.empty(rows, config.hidden, dtype=torch.int8, device=device)
        self.quant_o = torch.empty(rows, config.q_width, dtype=torch.int8, device=device)
        self.quant12 = torch.empty(rows, config.intermediate, dtype=torch.int8, device=device)
        self.scales = torch.empty(rows, dtype=torch.float32, device=device)
        self.maxima = torch.zeros(rows, dtype=torch.int32, device=device)
        self.decode_maxima = torch.zeros(2, dtype=torch.int32, device=device)  # one row: {max |attention|, max |act|}
        self.partial = torch.empty(rows, config.hidden, dtype=act, device=device)  # tensor parallel: O / down partial sums
        self.logits = None  # only the unfused path writes logits

    def first_rows(self, rows: int) -> "Workspace":
        """The same buffers cut down to their first `rows` rows (a shorter prompt in a workspace sized for the longest)."""
        if rows > self.rows:
            raise ValueError(f"workspace holds {self.rows} rows, {rows} asked for")
        view = object.__new__(Workspace)
        view.rows = rows
        for name, value in vars(self).items():
            if name == "rows":
                continue
            cut = isinstance(value, torch.Tensor) and name != "decode_maxima"
            setattr(view, name, value[:rows] if cut else value)
        return view


class Qwen3Runner:
    """GpuModel: owns the caches, the decode workspace, the control buffer and the captured decode graph.

    Decode launches may carry L2 prefetch hints for weights that a later projection streams (the reference's
    next-weight prefetch, src/gpu.rs:19-42).  Measured on a B200 (2.75 ms per token without hints): the down matrix
    hinted at the launch that quantizes the attention output gives 2.67 ms, at the quantize_with_max launch 2.68 ms;
    hinting the trailing gate / up rows at the attention launch costs time (2.77-2.91 ms).  Hence the defaults.

    unfused=True runs every projection with the one-thread-per-output kernel (VARIANT_NAIVE) and every fused step
    as its separate parts (swiglu then quantize; logits then selection); it exists to check that the fast kernels
    change nothing in a whole generation."""

    def __init__(self, weights: Qwen3Weights, unfused: bool = False, device="cuda", fold_quantizers: str = "none",
                 prefetch_rows: int = 0, prefetch_down_at: str = "quant", prefetch_o: bool = False, group=None,
                 fused_allreduce: bool = True, fold_attention_quantizer: bool = False, batch: int = 1,
                 peer_rows_times_ranks: int = 128, resident: bool | None = None, resident_exchange: bool = False):
        ops.init()
        if batch < 1:
            raise ValueError("batch must be at least 1")
        self.batch = batch  # sequences decoded side by side (generate_batch); 1 = the reference's single request
        self.group = group  # torch.distributed process group of the tensor-parallel ranks (weights.tp > 1)
        # decode: attention also writes the O projection's input codes (qwen3_attention_quantize).  Off: measured 2.69 ms per
        # token against 2.47 with the separate quantizer launch, whose latency programmatic launch already hides.
        self.fold_attention_quantizer = fold_attention_quantizer
        # Tensor parallel decode: O and down with the all-reduce fused in (tp.PeerLinear) instead of NCCL + `residual`.
        # The fused exchange sends every partial output to every rank as an 8-byte packet: rows * 4096 * 8 bytes * (ranks - 1)
        # per rank and call.  That beats NCCL's latency for decode-sized launches, but at 64 rows on 8 ranks it is 14.7 MB
        # per call against 0.5 MB of bf16 partials, so beyond rows * ranks = 128 the projection is followed by NCCL instead.
        self.peer_rows_times_ranks = peer_rows_times_ranks
        self.peer = None
        if weights.tp > 1 and fused_allreduce and not unfused:
            from .tp import PeerLinear

            self.peer = PeerLinear(group, max(16, min(batch, self.PEER_MAX_ROWS)) * weights.config.hidden)
        if weights.tp > 1 and fold_quantizers != "none":
            raise ValueError("folded quantizers are a single-GPU option")
        self.prefetch_rows = prefetch_rows
        self.prefetch_down_at = prefetch_down_at
        self.prefetch_o = prefetch_o
        self.fold_quantizers = fold_quantizers
        self.w = weights
        self.c = weights.config
        self.unfused = unfused
        self.device = device
        c = self.c
        # [sequence][position][kv head][128] per layer; k_cache / v_cache are sequence 0's caches (the single request)
        self.k_cache_all = [torch.zeros(batch, c.context, c.kv_heads, 128, dtype=torch.bfloat16, device=device) for _ in range(c.layers)]
        self.v_cache_all = [torch.zeros(batch, c.context, c.kv_heads, 128, dtype=torch.bfloat16, device=device) for _ in range(c.layers)]
        self.k_cache = [cache[0] for cache in self.k_cache_all]
        self.v_cache = [cache[0] for cache in self.v_cache_all]
        self.control = torch.zeros(2, dtype=torch.int32, device=device)   # {token, position}
        self.next = torch.zeros(1, dtype=torch.int32, device=device)
        self.decode = Workspace(c, 1, device, wide_gate_up=unfused)
        self.head_q = torch.empty(1, c.hidden, dtype=torch.int8, device=device)
        self.head_scale = torch.empty(1, dtype=torch.float32, device=device)
        self.head_x = torch.empty(1, c.hidden, dtype=torch.bfloat16, device=device)  # final norm row (bf16 head)
        self.head_rows = weights.head_bf16.shape[0] if weights.head_bf16 is not None else weights.head.n  # this rank's vocabulary rows
        self.logits = torch.empty(1, weights.full_config.vocab, dtype=torch.bfloat16, device=device) if unfused else None
        if weights.tp > 1:
            self.local_logits = torch.empty(1, self.head_rows, dtype=torch.bfloat16, device=device) if unfused else None
            self.local_best = torch.zeros(2, dtype=torch.int32, device=device)         # {token within the shard, value bits}
            self.all_best = torch.zeros(weights.tp, 2, dtype=torch.int32, device=device)
        self.graph = None
        # One-token decode: all layers of a step inside one resident kernel (ops.DecodePlan) instead of ten launches per
        # layer; bit-identical.  resident=None: on wherever the library supports the shape and the device.  Tensor parallel:
        # the same kernel on every rank's shard, O and down exchanging their partial outputs as packets over peer memory
        # inside it (needs fused_allreduce: the arithmetic is that of the fused exchange).  resident_exchange=True runs
        # that form on one GPU as a group of one (a test of the exchange code without a second device).
        self.plan = None
        self._exchange = None
        if resident is None:
            resident = os.environ.get("W8A8_RESIDENT_DECODE", "1") != "0"
        exchange = (weights.tp > 1 and fused_allreduce) or (weights.tp == 1 and resident_exchange)
        if resident and not unfused and fold_quantizers == "none" and (weights.tp == 1 or fused_allreduce):
            try:
                self.plan = ops.DecodePlan(weights.layers, self.k_cache, self.v_cache, c.hidden, c.q_heads, c.kv_heads, c.intermediate,
                                           c.eps, weights.rope)
                if exchange:
                    self._exchange = self._make_exchange(weights.tp, weights.rank, c.hidden)
                    self.plan.set_peers(*self._exchange[:2], weights.rank, weights.tp)
            except capi.W8A8Error as error:
                if error.status != 3:  # W8A8_ERR_UNSUPPORTED: this shape stays on the launch-per-operator path
                    raise
                self.plan = None
        self._host_control = torch.zeros(2, dtype=torch.int32).pin_memory()
        self._host_next = torch.zeros(1, dtype=torch.int32).pin_memory()
        # batched decode: one row per sequence
        self.batch_graph = None
        self.batch_ws = None
        if batch > 1 or os.environ.get("W8A8_BATCH_BUFFERS"):
            self._make_batch_buffers()

    PEER_MAX_ROWS = 64  # w8a8_linear_allreduce takes decode-sized launches only

    def _make_exchange(self, tp: int, rank: int, hidden: int):
        """Packet buffers of the resident decode kernel's exchanges: [2 halves][tp sources][hidden] packets of 8 bytes per
        rank, in symmetric memory when there are peers.  Returns (addresses by rank, seq word, what must stay alive)."""
        device = torch.device("cuda", torch.cuda.current_device())
        seq = torch.zeros(4, dtype=torch.int32, device=device)
        if tp == 1:
            buf = torch.zeros(2 * hidden * 2, dtype=torch.int32, device=device)
            return [buf.data_ptr()], seq, buf
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        buf = symm.empty(2 * tp * hidden * 2, dtype=torch.int32, device=device)
        handle = symm.rendezvous(buf, self.group.group_name if hasattr(self.group, "group_name") else self.group)
        buf.zero_()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        return [int(p) for p in handle.buffer_ptrs], seq, (buf, handle)

    def _make_batch_buffers(self) -> None:
        c, w, device, rows = self.c, self.w, self.device, self.batch
        self.batch_ws = Workspace(c, rows, device, wide_gate_up=self.unfused or rows > 4)
        self.batch_state = torch.zeros(2, rows, dtype=torch.int32, device=device)   # {token, position} per sequence
        self.tokens, self.positions = self.batch_state[0], self.batch_state[1]
        self.next_tokens = torch.zeros(rows, dtype=torch.int32, device=device)
        self.attention_ws = ops.attention_batched_workspace(rows, c.q_heads, c.kv_heads, device)
        self.batch_head_q = torch.empty(rows, c.hidden, dtype=torch.int8, device=device)
        self.batch_head_scale = torch.empty(rows, dtype=torch.float32, device=device)
        if w.head is None:
            raise ValueError("batched decode needs the W8A8 head (the bf16 head kernel serves one row per launch)")
        stored = self.unfused or rows > 16  # the fused head + selection kernel takes at most 16 rows
        self.batch_logits = torch.empty(rows, w.head.n, dtype=torch.bfloat16, device=device) if stored else None
        if w.tp > 1:
            self.batch_best = torch.zeros(2, rows, dtype=torch.int32, device=device)        # local {tokens, value bits}
            self.batch_all_best = torch.zeros(w.tp, 2, rows, dtype=torch.int32, device=device)
        self._host_state = torch.zeros(2, rows, dtype=torch.int32).pin_memory()
        self._host_next_tokens = torch.zeros(rows, dtype=torch.int32).pin_memory()

    # -- one forward pass: queues kernels only ------------------------------------------------------------
    def forward(self, ws: Workspace, ids: torch.Tensor, slot: int = 0, batched: bool = False) -> None:
        """One pass over `ws.rows` rows.  batched=False: the rows are consecutive tokens of the sequence in cache `slot`,
        the first at position control[1] (prefill, or one decode step of the single request).  batched=True: row r is the
        newest token of sequence r at position positions[r] (one decode step of every sequence; `ids` is self.tokens)."""
        c, w = self.c, self.w
        variant = capi.VARIANT_NAIVE if self.unfused else capi.VARIANT_AUTO
        rows = ws.rows
        q4, qo = ws.quant4, ws.quant_o
        inter = c.intermediate
        single = rows == 1 and not batched  # the reference's decode step: hints and folded quantizers apply
        ops.embedding(ids, w.embedding, ws.hidden)
        if single and self.plan is not None and slot == 0:
            self.plan.run(ws.hidden, self.control)
            return self._head(ws)
        if single and self.fold_quantizers != "none" and not self.unfused:
            self._decode_layers(ws)
            return self._head(ws)
        for index, layer in enumerate(w.layers):
            k_cache, v_cache = self.k_cache_all[index][slot], self.v_cache_all[index][slot]
            ops.norm_quantize(ws.hidden, layer.norm1, None, q4, ws.scales, ws.maxima, c.eps)
            ops.linear_quantized(q4, ws.scales, layer.qkv, ws.qkv, variant)
            if batched:
                ops.prepare_qk_batched(ws.qkv, c.q_heads, c.kv_heads, layer.qnorm, layer.knorm, w.rope, self.positions,
                                       self.k_cache_all[index], self.v_cache_all[index])
                ops.attention_batched(ws.qkv, c.q_heads, c.kv_heads, self.k_cache_all[index], self.v_cache_all[index],
                                      self.positions, ws.attention, self.attention_ws)
                ops.quantize(ws.attention, qo, ws.scales)
                self._project_residual(ws, qo, layer.o, ws.hidden, ws.residual, variant)
                self._mlp(ws, layer, variant, single)
                continue
            ops.prepare_qk(ws.qkv, c.q_heads, c.kv_heads, layer.qnorm, layer.knorm, w.rope, self.control, k_cache, v_cache)
            if rows == 1 and self.prefetch_rows and not self.unfused:
                # Decode: the attention launch also pulls the last rows of gate and up towards L2; the gate/up kernel's
                # first wave of CTAs fetches the leading rows by itself before its dependency wait.
                first = max(0, inter - self.prefetch_rows) * c.hidden
                ops.prefetch_hint(layer.gate_up.w, first, self.prefetch_rows * c.hidden)
                ops.prefetch_hint(layer.gate_up.w, inter * c.hidden + first, self.prefetch_rows * c.hidden)
            if rows == 1 and self.prefetch_o and not self.unfused:
                ops.prefetch_hint(layer.o.w)
            if rows == 1 and self.prefetch_down_at == "attention" and not self.unfused:
                ops.prefetch_hint(layer.down.w)
            if rows == 1 and self.fold_attention_quantizer and not self.unfused:
                if self.prefetch_down_at == "quant":  # the quantizer launch is gone: the hint rides on the attention launch
                    ops.prefetch_hint(layer.down.w)
                ops.attention_quantize(ws.qkv, c.q_heads, c.kv_heads, k_cache, v_cache, self.control, ws.attention, qo, ws.scales)
            else:
                ops.attention(ws.qkv, c.q_heads, c.kv_heads, k_cache, v_cache, self.control, ws.attention)
                if rows == 1 and self.prefetch_down_at == "quant" and not self.unfused:
                    ops.prefetch_hint(layer.down.w)
                ops.quantize(ws.attention, qo, ws.scales)
            self._project_residual(ws, qo, layer.o, ws.hidden, ws.residual, variant)
            if rows == 1 and self.prefetch_down_at == "norm2" and not self.unfused:
                ops.prefetch_hint(layer.down.w)
            self._mlp(ws, layer, variant, single)
        if batched:
            self._head_rows(ws)
        else:
            self._head(ws)

    def _mlp(self, ws: Workspace, layer: Layer, variant: int, single: bool) -> None:
        """norm_quantize -> gate / up projections -> SwiGLU -> quantize -> down projection + residual."""
        c = self.c
        rows, inter, q4 = ws.rows, c.intermediate, ws.quant4
        ops.norm_quantize(ws.residual, layer.norm2, None, q4, ws.scales, ws.maxima, c.eps)
        if self.unfused:
            ops.linear_quantized(q4, ws.scales, layer.gate_up, ws.gate_up, variant)
            ops.swiglu(ws.gate_up[:, :inter], ws.gate_up[:, inter:], ws.act, None)
            ops.quantize(ws.act, ws.quant12, ws.scales)
        elif rows == 1 or (rows <= 4 and ws.gate_up is None):
            # few rows: gate and up share every activation load and the SwiGLU is the projection's epilogue
            ops.linear_swiglu(q4, ws.scales, layer.gate, layer.up, None, None, ws.act, ws.maxima)
            if single and self.prefetch_down_at == "qwm":
                ops.prefetch_hint(layer.down.w)
            ops.quantize_with_max(ws.act, ws.maxima, ws.quant12, ws.scales)
        else:
            ops.linear_quantized(q4, ws.scales, layer.gate_up, ws.gate_up, variant)
            ops.swiglu_quantize(ws.gate_up[:, :inter], ws.gate_up[:, inter:], ws.quant12, ws.scales)
        self._project_residual(ws, ws.quant12, layer.down, ws.residual, ws.hidden, variant)

    def _project_residual(self, ws: Workspace, q: torch.Tensor, matrix, residual_in: torch.Tensor, combined: torch.Tensor,
                          variant: int) -> None:
        """combined = bf16(residual_in + projection).  One GPU: the residual sum is the projection's epilogue.  Tensor
        parallel (O and down own a slice of the input channels): bf16 partial projection, all-reduce, then `residual`."""
        if self.w.tp == 1:
            ops.linear_residual(q, ws.scales, matrix, None, residual_in, combined, variant)
            return
        if (self.peer is not None and ws.rows * matrix.n <= self.peer.slot and ws.rows <= self.PEER_MAX_ROWS
                and ws.rows * self.w.tp <= self.peer_rows_times_ranks):
            self.peer.linear_residual(q, ws.scales, matrix, None, residual_in, combined)
            return
        import torch.distributed as dist

        ops.linear_quantized(q, ws.scales, matrix, ws.partial, variant)
        dist.all_reduce(ws.partial, op=dist.ReduceOp.SUM, group=self.group)
        ops.residual(residual_in, ws.partial, combined)

    def _decode_layers(self, ws: Workspace) -> None:
        """One row, with quantizers folded into the projections that consume them: "with_max" folds the quantizers of
        the O and down projections (their maxima come from the producers: attention and the SwiGLU epilogue), "all"
        also the two RMSNorm quantizers (six launches per layer instead of ten)."""
        c, w = self.c, self.w
        att_max, act_max = ws.decode_maxima[0:1], ws.decode_maxima[1:2]
        fold_norm = self.fold_quantizers == "all"
        for index, layer in enumerate(w.layers):
            if fold_norm:
                ops.quantize_linear(ws.hidden, layer.qkv, ws.qkv, gain=layer.norm1, eps=c.eps, maxima_reset=ws.decode_maxima)
            else:
                ops.norm_quantize(ws.hidden, layer.norm1, None, ws.quant4, ws.scales, att_max, c.eps)
                ops.linear_quantized(ws.quant4, ws.scales, layer.qkv, ws.qkv)
            ops.prepare_qk(ws.qkv, c.q_heads, c.kv_heads, layer.qnorm, layer.knorm, w.rope, self.control,
                           self.k_cache[index], self.v_cache[index])
            ops.attention(ws.qkv, c.q_heads, c.kv_heads, self.k_cache[index], self.v_cache[index], self.control, ws.attention,
                          att_max)
            ops.quantize_linear(ws.attention, layer.o, None, maxima_in=att_max, residual_in=ws.hidden, combined=ws.residual)
            if fold_norm:
                ops.quantize_linear_swiglu(ws.residual, layer.gate, layer.up, ws.act, act_max, gain=layer.norm2, eps=c.eps)
            else:
                ops.norm_quantize(ws.residual, layer.norm2, None, ws.quant4, ws.scales, act_max, c.eps)
                ops.linear_swiglu(ws.quant4, ws.scales, layer.gate, layer.up, None, None, ws.act, act_max)
            ops.quantize_linear(ws.act, layer.down, None, maxima_in=act_max, residual_in=ws.residual, combined=ws.hidden)

    def _head(self, ws: Workspace) -> None:
        c, w = self.c, self.w
        rows = ws.rows
        variant = capi.VARIANT_NAIVE if self.unfused else capi.VARIANT_AUTO
        last = ws.hidden[rows - 1:rows]
        bf16_head = w.head_bf16 is not None
        # the final norm; with a bf16 head its output row is what the head multiplies (the reference's `norm`, src/gpu.rs:798)
        ops.norm_quantize(last, w.final_gain, self.head_x if bf16_head else None, self.head_q, self.head_scale, None, c.eps)
        if w.tp == 1:
            if bf16_head and self.unfused:
                ops.head_bf16(self.head_x, w.head_bf16, logits=self.logits)
            elif bf16_head:
                ops.head_bf16(self.head_x, w.head_bf16, token=self.next)
            elif self.unfused:
                ops.linear_quantized(self.head_q, self.head_scale, w.head, self.logits, variant)
            else:
                ops.linear_argmax(self.head_q, self.head_scale, w.head, self.next)
            return
        # vocabulary split: every rank projects its rows; logits (unfused) or (token, value) candidates are gathered
        import torch.distributed as dist

        if self.unfused:
            if bf16_head:
                ops.head_bf16(self.head_x, w.head_bf16, logits=self.local_logits)
            else:
                ops.linear_quantized(self.head_q, self.head_scale, w.head, self.local_logits, variant)
            dist.all_gather_into_tensor(self.logits.view(-1), self.local_logits.view(-1), group=self.group)
            return
        if bf16_head:
            ops.head_bf16(self.head_x, w.head_bf16, token=self.local_best[0:1], value=self.local_best[1:2].view(torch.float32))
        else:
            ops.linear_argmax(self.head_q, self.head_scale, w.head, self.local_best[0:1], self.local_best[1:2].view(torch.float32))
        dist.all_gather_into_tensor(self.all_best.view(-1), self.local_best, group=self.group)
        # device-side selection over the ranks' candidates (no host synchronisation: this runs inside the captured step)
        ops.merge_candidates(self.all_best.view(w.tp, 2, 1), self.head_rows, self.next)

    def _head_rows(self, ws: Workspace) -> None:
        """Final norm, head projection and greedy selection for every row (batched decode): next_tokens[r]."""
        c, w = self.c, self.w
        rows = ws.rows
        variant = capi.VARIANT_NAIVE if self.unfused else capi.VARIANT_AUTO
        ops.norm_quantize(ws.hidden, w.final_gain, None, self.batch_head_q, self.batch_head_scale, None, c.eps)
        if w.tp == 1:
            token, value = self.next_tokens, None
        else:
            token, value = self.batch_best[0], self.batch_best[1].view(torch.float32)
        if self.batch_logits is None:
            ops.linear_argmax(self.batch_head_q, self.batch_head_scale, w.head, token, value)
        else:  # more rows than the fused kernel takes: store this rank's logits, then `select_token` per row
            ops.linear_quantized(self.batch_head_q, self.batch_head_scale, w.head, self.batch_logits, variant)
            ops.select_token(self.batch_logits, token, value)
        if w.tp > 1:
            import torch.distributed as dist

            dist.all_gather_into_tensor(self.batch_all_best.view(-1), self.batch_best.view(-1), group=self.group)
            ops.merge_candidates(self.batch_all_best, w.head.n, self.next_tokens)

    def _select_unfused(self) -> int:
        """select_token (src/kernels.rs:2191-2231) on the written logits: largest value, lowest index."""
        logits = self.logits[0].float()
        if not bool(torch.isfinite(logits).all()):
            return 0xFFFFFFFF
        return int((logits == logits.max()).nonzero()[0, 0])

    def capture_decode(self) -> None:
        """Capture one decode step (src/gpu.rs:303-333).  Everything it reads that changes between steps lives in
        the control buffer and the caches."""
        ops.set_programmatic_launch(True)
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self.control.zero_()
            self.forward(self.decode, self.control)  # warm-up outside the capture
        stream.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=stream):
            self.forward(self.decode, self.control)
        torch.cuda.current_stream().wait_stream(stream)
        ops.set_programmatic_launch(False)

    def capture_batch_decode(self) -> None:
        """One decode step of every sequence, captured once: what changes between steps lives in `batch_state`
        ({token, position} per sequence) and the caches."""
        ops.set_programmatic_launch(True)
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self.batch_state.zero_()
            self.forward(self.batch_ws, self.tokens, batched=True)  # warm-up outside the capture
        stream.synchronize()
        self.batch_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.batch_graph, stream=stream):
            self.forward(self.batch_ws, self.tokens, batched=True)
        torch.cuda.current_stream().wait_stream(stream)
        ops.set_programmatic_launch(False)

    def generate_batch(self, prompts, max_tokens: int, use_graph: bool = True):
        """Greedy generation for `batch` independent sequences side by side: each prompt is prefilled on its own into its
        sequence's caches (the reference's first step, src/gpu.rs:893-901, once per sequence), then every decode step
        advances all sequences by one token in ONE pass of `batch` rows -- the sequences may have any mix of context
        lengths.  Returns (one token list per sequence, seconds per step; the first entry is the whole prefill phase)."""
        import time

        c = self.c
        if self.batch_ws is None:
            self._make_batch_buffers()
        if len(prompts) != self.batch:
            raise ValueError(f"this runner decodes {self.batch} sequences side by side, {len(prompts)} prompts given")
        for prompt in prompts:
            if not prompt or len(prompt) + max_tokens > c.context:
                raise ValueError("every prompt must be non-empty and prompt + max_tokens must fit the context")
        if use_graph and not self.unfused and self.batch_graph is None:
            self.capture_batch_decode()
        torch.cuda.synchronize()
        start = time.perf_counter()
        longest = Workspace(c, max(len(p) for p in prompts), self.device)
        ids = torch.empty(longest.rows, dtype=torch.int32, device=self.device)
        generated = []
        for slot, prompt in enumerate(prompts):
            self._host_control[0] = 0
            self._host_control[1] = 0
            self.control.copy_(self._host_control, non_blocking=True)
            ids[:len(prompt)].copy_(torch.tensor(list(prompt), dtype=torch.int32), non_blocking=False)
            self.forward(longest.first_rows(len(prompt)), ids[:len(prompt)], slot=slot)
            token = self._read_next()
            if token == 0xFFFFFFFF:
                raise RuntimeError("nonfinite or empty logits")
            generated.append([token])
        del longest
        seconds = [time.perf_counter() - start]
        positions = [len(p) for p in prompts]
        for _ in range(1, max_tokens):
            start = time.perf_counter()
            for r in range(self.batch):
                self._host_state[0, r] = generated[r][-1]
                self._host_state[1, r] = positions[r]
            self.batch_state.copy_(self._host_state, non_blocking=True)
            if self.batch_graph is not None and use_graph and not self.unfused:
                self.batch_graph.replay()
            else:
                self.forward(self.batch_ws, self.tokens, batched=True)
            self._host_next_tokens.copy_(self.next_tokens, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            seconds.append(time.perf_counter() - start)
            for r in range(self.batch):
                token = int(self._host_next_tokens[r]) & 0xFFFFFFFF
                if token == 0xFFFFFFFF:
                    raise RuntimeError("nonfinite or empty logits")
                generated[r].append(token)
                positions[r] += 1
        return generated, seconds

    def _read_next(self) -> int:
        if self.unfused:
            return self._select_unfused()
        self._host_next.copy_(self.next, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return int(self._host_next[0]) & 0xFFFFFFFF

    def generate(self, prompt_ids, max_tokens: int, use_graph: bool = True, stop_ids=()):
        """GpuModel::generate (src/gpu.rs:818-929): prefill the prompt, then one token per step.  Returns
        (token ids, seconds per step); the first step is the prefill."""
        import time

        c = self.c
        if not prompt_ids or len(prompt_ids) + max_tokens > c.context:
            raise ValueError("prompt must be non-empty and prompt + max_tokens must fit the context")
        if use_graph and not self.unfused and self.graph is None:
            self.capture_decode()
        torch.cuda.synchronize()
        prompt = torch.tensor(list(prompt_ids), dtype=torch.int32).pin_memory()
        prefill = Workspace(c, len(prompt_ids), self.device)
        ids = torch.empty(len(prompt_ids), dtype=torch.int32, device=self.device)
        generated, seconds = [], []
        position, rows, token = 0, len(prompt_ids), 0
        for step in range(max_tokens):
            start = time.perf_counter()
            self._host_control[0] = token
            self._host_control[1] = position
            self.control.copy_(self._host_control, non_blocking=True)
            if step == 0:
                ids.copy_(prompt, non_blocking=True)
                self.forward(prefill, ids)
            elif self.graph is not None and use_graph and not self.unfused:
                self.graph.replay()
            else:
                self.forward(self.decode, self.control)
            token = self._read_next()
            seconds.append(time.perf_counter() - start)
            if token == 0xFFFFFFFF:
                raise RuntimeError("nonfinite or empty logits")
            generated.append(token)
            if token in stop_ids:
                break
            position += rows
            rows = 1
        return generated, seconds
