"""Helpers shared by the GPU parity tests: numpy <-> device tensors, synthetic inputs."""
from __future__ import annotations

import numpy as np

from oracle import oracle


def to_dev(a: np.ndarray, dtype: str = "raw"):
    """numpy -> cuda tensor.  dtype 'bf16' stores bf16-representable float32 values as torch.bfloat16;
    'f32' keeps the reference's f32 carrier; 'raw' keeps the numpy dtype."""
    import torch

    if dtype == "bf16":
        bits = oracle.bf16_bits(a).astype(np.int16)
        return torch.from_numpy(bits).cuda().view(torch.bfloat16).reshape(a.shape)
    if dtype == "f32":
        return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def to_host(t) -> np.ndarray:
    """cuda tensor -> numpy; bf16 tensors come back as float32 values."""
    import torch

    if t.dtype == torch.bfloat16:
        bits = t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        return oracle.from_bf16_bits(bits).reshape(t.shape)
    return t.cpu().numpy()


def empty_act(shape, dtype: str, fill: float | None = float("nan")):
    """Output buffer, poisoned so that an unwritten element cannot pass for a result."""
    import torch

    td = torch.bfloat16 if dtype == "bf16" else torch.float32
    t = torch.empty(shape, dtype=td, device="cuda")
    if fill is not None:
        t.fill_(fill)
    return t


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def gate(actual, expected):
    """The reference's numeric gate (src/conformance.rs:658-674; docs/qwen3-8b-w8a8/coverage.md:28):
    |err| <= 2e-4 + 0.01*|expected| and relative L2 <= 0.005."""
    a = np.asarray(actual, dtype=np.float64).ravel()
    e = np.asarray(expected, dtype=np.float64).ravel()
    assert np.all(np.abs(a - e) <= 2e-4 + 0.01 * np.abs(e)), float(np.abs(a - e).max())
    denom = np.linalg.norm(e)
    if denom > 0:
        assert np.linalg.norm(a - e) / denom <= 0.005


def ulp_distance_bf16(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in bf16 ulps between bf16-representable float32 arrays (sign-magnitude aware)."""
    def key(x):
        u = (bits(x) >> np.uint32(16)).astype(np.int64)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(a) - key(b))


# ---- seeded synthetic tensors with the value distributions of the benchmark configs -------------

def synth_activations(rng: np.random.Generator, M: int, K: int) -> np.ndarray:
    """bf16(N(0,1)) with 8 seeded outlier channels scaled x20 (before bf16 rounding)."""
    x = rng.standard_normal((M, K), dtype=np.float32)
    cols = rng.choice(K, size=8, replace=False)
    x[:, cols] *= 20.0
    return oracle.bf16(x)


def synth_weights(rng: np.random.Generator, N: int, K: int):
    """fp32 N(0,0.02) quantized per output channel (tools/prepare.py:79-81) -> (int8 [N,K], f32 [N])."""
    w = rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
    s = np.maximum(np.abs(w).max(axis=1), np.float32(1e-8)) / np.float32(127)
    q = np.clip(np.rint(w / s[:, None]), -127, 127).astype(np.int8)
    return q, s.astype(np.float32)


def synth_gamma(rng: np.random.Generator, K: int) -> np.ndarray:
    return oracle.bf16((1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32))
