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
