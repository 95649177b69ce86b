"""Tensor-parallel sharding of the W8A8 linear layer inside one box (host-side plumbing only).

The reference has no multi-GPU code (`CudaContext::new(0)`, crates/inferrous-qwen3/src/gpu.rs:248;
tensor parallelism is deferred in docs/plans/production.md:232), so this layout is this library's own:

  column split  QKV, gate_up, lm_head: each rank owns N/tp output channels; no communication
                (gate and up are split identically so SwiGLU stays local; QKV is split by head).
  row split     O, down: each rank owns K/tp input channels of every output, quantizes its slice of the
                activations with its LOCAL absmax, applies its own a_scale in the epilogue, and the bf16
                partial outputs [M,N] are summed by one all-reduce.

One process per GPU; `torch.distributed` (NCCL on GPUs, gloo in the CPU tests) carries the all-reduce.
"""
from __future__ import annotations

ROW_SPLIT = frozenset({"o", "down"})


def shard_shape(name: str, K: int, N: int, tp: int) -> tuple[int, int]:
    """(K, N) of one rank's shard."""
    if tp == 1:
        return K, N
    if name in ROW_SPLIT:
        if K % (128 * tp):
            raise ValueError(f"{name}: K={K} cannot be split {tp} ways in multiples of 128")
        return K // tp, N
    if N % tp:
        raise ValueError(f"{name}: N={N} is not divisible by tp={tp}")
    return K, N // tp


def shard_weight(name: str, w, w_scale, rank: int, tp: int):
    """Slice a full [N,K] weight (+ per-channel scales) for `rank`.  Works on numpy arrays and torch tensors.
    Row-split shards keep every output channel, so they keep the full scale vector."""
    N, K = w.shape
    k, n = shard_shape(name, K, N, tp)
    if name in ROW_SPLIT:
        return w[:, rank * k:(rank + 1) * k], w_scale
    return w[rank * n:(rank + 1) * n], w_scale[rank * n:(rank + 1) * n]


def shard_activation(name: str, x, rank: int, tp: int):
    """The slice of the activations [M,K] a rank multiplies: all of it for column splits, its K slice for row splits."""
    if tp == 1 or name not in ROW_SPLIT:
        return x
    k = x.shape[1] // tp
    return x[:, rank * k:(rank + 1) * k]


def needs_all_reduce(name: str, tp: int) -> bool:
    return tp > 1 and name in ROW_SPLIT


def all_reduce_sum(y, group=None):
    """In-place sum of the partial outputs over the tensor-parallel group (bf16 on GPUs)."""
    import torch.distributed as dist

    dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y


class PeerAllReduce:
    """One-shot all-reduce of decode-sized partial outputs over peer memory (w8a8_tp_allreduce).

    Each rank owns a staging buffer in symmetric memory ([2 halves][tp slots][slot_elems]) and a flag pad; every
    rank sees every other rank's buffer and pad through NVLink.  `all_reduce(partial, out)` queues ONE kernel on the
    current stream: push to all ranks, bounded wait, sum in rank order (f32) -> bf16.  Capturable in a CUDA graph.
    Falls back to nothing: if symmetric memory cannot be set up, construction raises and the caller uses NCCL."""

    def __init__(self, group, slot_elems: int, dtype=None):
        import ctypes as C

        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import capi

        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.dtype = dtype or torch.bfloat16
        self.slot_elems = (slot_elems + 127) // 128 * 128
        dev = torch.device("cuda", torch.cuda.current_device())
        # one symmetric allocation: 256 bytes of arrival counters (the library's own, not torch's signal pad),
        # then the two halves of the staging area
        flag_elems = 256 // torch.empty((), dtype=self.dtype).element_size()
        self.buf = symm.empty(flag_elems + 2 * self.tp * self.slot_elems, dtype=self.dtype, device=dev)
        self.handle = symm.rendezvous(self.buf, group.group_name if hasattr(group, "group_name") else group)
        self.buf.zero_()
        self.seq = torch.zeros(4, dtype=torch.int32, device=dev)
        self._flags = (C.c_void_p * self.tp)(*[int(p) for p in self.handle.buffer_ptrs])
        self._bufs = (C.c_void_p * self.tp)(*[int(p) + 256 for p in self.handle.buffer_ptrs])
        self._lib = capi.load()
        self._capi = capi
        torch.cuda.synchronize()
        dist.barrier(group)

    def all_reduce(self, partial, out=None):
        import ctypes as C

        import torch

        out = partial if out is None else out
        n = partial.numel()
        code = 0 if partial.dtype == torch.bfloat16 else 1
        st = self._lib.w8a8_tp_allreduce(C.c_void_p(partial.data_ptr()), C.c_void_p(out.data_ptr()), n, code, self._bufs,
                                         self._flags, C.c_void_p(self.seq.data_ptr()), self.rank, self.tp, self.slot_elems,
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream))
        self._capi.check(st, "w8a8_tp_allreduce")
        return out


# ---- whole-model sharding: which rows / columns of the concatenated matrices a rank owns ---------------------

def qkv_rows(q_heads: int, kv_heads: int, rank: int, tp: int, head_dim: int = 128):
    """Row ranges (start, stop) of the concatenated Q|K|V matrix owned by `rank`: its query heads, then the key heads and
    value heads they attend to.  Heads are dealt in contiguous blocks, so query head h keeps key/value head h // group."""
    if q_heads % tp or kv_heads % tp:
        raise ValueError(f"{q_heads} query / {kv_heads} key-value heads cannot be split {tp} ways")
    ql, kl = q_heads // tp * head_dim, kv_heads // tp * head_dim
    q_width, kv_width = q_heads * head_dim, kv_heads * head_dim
    return [(rank * ql, (rank + 1) * ql), (q_width + rank * kl, q_width + (rank + 1) * kl),
            (q_width + kv_width + rank * kl, q_width + kv_width + (rank + 1) * kl)]


def gate_up_rows(intermediate: int, rank: int, tp: int):
    """Row ranges of the concatenated gate|up matrix owned by `rank` (the same channels of both, so SwiGLU stays local)."""
    if intermediate % (128 * tp):
        raise ValueError(f"intermediate width {intermediate} cannot be split {tp} ways in multiples of 128")
    il = intermediate // tp
    return [(rank * il, (rank + 1) * il), (intermediate + rank * il, intermediate + (rank + 1) * il)]


def take_rows(w, w_scale, ranges):
    """Concatenate row ranges of a weight [N,K] and of its per-channel scales (numpy arrays or torch tensors)."""
    if hasattr(w, "numpy") or type(w).__module__.startswith("torch"):
        import torch

        return (torch.cat([w[a:b] for a, b in ranges]).contiguous(), torch.cat([w_scale[a:b] for a, b in ranges]).contiguous())
    import numpy as np

    return np.concatenate([w[a:b] for a, b in ranges]), np.concatenate([w_scale[a:b] for a, b in ranges])


class PeerLinear:
    """Row-split projections with the all-reduce fused in (w8a8_linear_allreduce): the GEMV's epilogue sends its partial
    output to every rank as tagged 8-byte packets over NVLink and a small consumer kernel sums them in rank order and adds
    the residual.  Owns the packet buffer in symmetric memory ([2 halves][tp sources][slot] packets per rank) and the
    call counter.  Decode-sized launches only (rows * output channels <= slot_packets).  Capturable in a CUDA graph."""

    def __init__(self, group, slot_packets: int):
        import ctypes as C

        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import capi

        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.slot = int(slot_packets)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buf = symm.empty(2 * self.tp * self.slot * 2, dtype=torch.int32, device=dev)  # 8 bytes per packet
        self.handle = symm.rendezvous(self.buf, group.group_name if hasattr(group, "group_name") else group)
        self.buf.zero_()
        self.seq = torch.zeros(4, dtype=torch.int32, device=dev)
        self._peers = (C.c_void_p * self.tp)(*[int(p) for p in self.handle.buffer_ptrs])
        self._lib = capi.load()
        self._capi = capi
        torch.cuda.synchronize()
        dist.barrier(group)

    def linear_residual(self, q, scale, matrix, out, residual_in, combined):
        """combined = bf16(residual_in + bf16(sum over ranks of the partial projections)); `out` (the sum) and the
        residual pair are both optional, at least one is required."""
        import ctypes as C

        import torch

        ref = combined if combined is not None else out
        code = 0 if ref.dtype == torch.bfloat16 else 1
        ptr = lambda t: None if t is None else C.c_void_p(t.data_ptr())
        st = self._lib.w8a8_linear_allreduce(ptr(q), ptr(scale), matrix.handle, q.shape[0], ptr(residual_in), ptr(out), ptr(combined),
                                             code, self._peers, ptr(self.seq), self.rank, self.tp, self.slot,
                                             C.c_void_p(torch.cuda.current_stream().cuda_stream))
        self._capi.check(st, "w8a8_linear_allreduce")
