"""numpy front-end to the plain-C CPU oracle (oracle/w8a8_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of bench.py.  The product package never imports this module.

Activation tensors are float32 arrays holding bf16-representable values, which
is also how the reference stores them (src/gpu.rs:16 `type Buffer = DeviceBuffer<f32>`).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "libw8a8_oracle.so"


def build(force: bool = False) -> Path:
    """Compile the oracle with gcc (a few hundred ms)."""
    src_time = max((_HERE / n).stat().st_mtime for n in ("w8a8_oracle.c", "w8a8_oracle.h", "Makefile"))
    if force or not _SO.exists() or _SO.stat().st_mtime < src_time:
        subprocess.run(["make", "-C", str(_HERE), "-B"], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_SO))
        vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
        L.oracle_bf16.restype = f
        L.oracle_bf16.argtypes = [f]
        L.oracle_round_i8_many.argtypes = [vp, vp, sz]
        L.oracle_quantize.argtypes = [vp, i, i, vp, vp]
        L.oracle_quantize_with_max.argtypes = [vp, vp, i, i, vp, vp]
        L.oracle_rmsnorm.argtypes = [vp, vp, f, i, i, vp]
        L.oracle_swiglu.argtypes = [vp, vp, sz, vp, vp]
        L.oracle_residual.argtypes = [vp, vp, sz, vp]
        L.oracle_linear_acc.argtypes = [vp, vp, i, i, i, vp, i]
        L.oracle_epilogue.argtypes = [vp, vp, vp, i, i, vp]
        L.oracle_linear.argtypes = [vp, vp, vp, vp, i, i, i, vp, vp, vp, i]
        L.oracle_weight_quantize.argtypes = [vp, i, i, vp, vp]
        L.oracle_hw_threads.restype = i
        for name in ("oracle_round_i8_many", "oracle_quantize", "oracle_quantize_with_max", "oracle_rmsnorm",
                     "oracle_swiglu", "oracle_residual", "oracle_linear_acc", "oracle_epilogue", "oracle_linear",
                     "oracle_weight_quantize"):
            getattr(L, name).restype = None
        _lib = L
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int8)


def hw_threads() -> int:
    return lib().oracle_hw_threads()


def bf16(x) -> np.ndarray:
    """f32 -> nearest-even bf16, kept as f32 (src/kernels.rs:12-15), vectorised in numpy."""
    u = _f32(x).view(np.uint32)
    u = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return u.view(np.float32)


def bf16_bits(x) -> np.ndarray:
    """bf16 storage bits (uint16) of bf16-representable float32 values."""
    return (_f32(x).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_i8(x) -> np.ndarray:
    x = _f32(x).ravel()
    out = np.empty(x.size, np.int8)
    lib().oracle_round_i8_many(_p(x), _p(out), x.size)
    return out


def quantize(x):
    x = _f32(x)
    M, K = x.shape
    q = np.empty((M, K), np.int8)
    s = np.empty((M,), np.float32)
    lib().oracle_quantize(_p(x), M, K, _p(q), _p(s))
    return q, s


def quantize_with_max(x, maxima_bits):
    x = _f32(x)
    M, K = x.shape
    mb = np.ascontiguousarray(maxima_bits, dtype=np.uint32)
    q = np.empty((M, K), np.int8)
    s = np.empty((M,), np.float32)
    lib().oracle_quantize_with_max(_p(x), _p(mb), M, K, _p(q), _p(s))
    return q, s


def rmsnorm(x, gain, eps: float = 1e-6):
    x = _f32(x)
    g = _f32(gain)
    M, K = x.shape
    y = np.empty((M, K), np.float32)
    lib().oracle_rmsnorm(_p(x), _p(g), eps, M, K, _p(y))
    return y


def swiglu(gate, up):
    """Returns (act, absmax_bits) over the whole flattened input (one row in decode)."""
    g = _f32(gate)
    u = _f32(up)
    act = np.empty(g.shape, np.float32)
    mx = np.zeros(1, np.uint32)
    lib().oracle_swiglu(_p(g), _p(u), g.size, _p(act), _p(mx))
    return act, int(mx[0])


def residual(a, b):
    a = _f32(a)
    b = _f32(b)
    out = np.empty(a.shape, np.float32)
    lib().oracle_residual(_p(a), _p(b), a.size, _p(out))
    return out


def linear_acc(q, w, threads: int = 0):
    q = _i8(q)
    w = _i8(w)
    M, K = q.shape
    N, K2 = w.shape
    assert K == K2
    acc = np.empty((M, N), np.int32)
    lib().oracle_linear_acc(_p(q), _p(w), M, N, K, _p(acc), threads)
    return acc


def epilogue(acc, asc, ws):
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    M, N = acc.shape
    asc = _f32(asc).reshape(M)
    ws = _f32(ws).reshape(N)
    y = np.empty((M, N), np.float32)
    lib().oracle_epilogue(_p(acc), _p(asc), _p(ws), M, N, _p(y))
    return y


def linear(q, asc, w, ws, residual_in=None, threads: int = 0):
    """Returns y, or (y, combined) when residual_in is given."""
    q = _i8(q)
    w = _i8(w)
    M, K = q.shape
    N = w.shape[0]
    asc = _f32(asc).reshape(M)
    ws = _f32(ws).reshape(N)
    y = np.empty((M, N), np.float32)
    if residual_in is None:
        lib().oracle_linear(_p(q), _p(asc), _p(w), _p(ws), M, N, K, None, _p(y), None, threads)
        return y
    r = _f32(residual_in).reshape(M, N)
    comb = np.empty((M, N), np.float32)
    lib().oracle_linear(_p(q), _p(asc), _p(w), _p(ws), M, N, K, _p(r), _p(y), _p(comb), threads)
    return y, comb


def weight_quantize(w):
    w = _f32(w)
    N, K = w.shape
    q = np.empty((N, K), np.int8)
    s = np.empty((N,), np.float32)
    lib().oracle_weight_quantize(_p(w), N, K, _p(q), _p(s))
    return q, s


# ---- the operators around the linear layers (numpy; float32 operations are separately rounded) ------------

def embedding(ids, table_bits):
    """src/kernels.rs:335-345: out[r] = widen(table[ids[r]]); table holds bf16 bit patterns."""
    return from_bf16_bits(np.asarray(table_bits, np.uint16)[np.asarray(ids, np.int64)])


def rope(x, table, position: int):
    """src/kernels.rs:1444-1468.  x: [rows, heads, 128] float32; table: [positions, 128] (64 cosines, 64 sines);
    row r is rotated with table[position + r]."""
    x = _f32(x)
    rows = x.shape[0]
    t = _f32(table)[position:position + rows]
    c = t[:, None, :64]
    s = t[:, None, 64:]
    a, b = x[..., :64], x[..., 64:]
    first = bf16(a * c + (-(b * s)))
    second = bf16(b * c + a * s)
    return np.concatenate([first, second], -1)


def head_norm(x, gain, eps: float = 1e-6, inv_ulps: int = 0):
    """RMSNorm of width 128 as norm_rope / prepare_qk compute it (src/kernels.rs:1304-1331): squares, the first tree
    level (p[t] + p[t+64]) + (p[t+32] + p[t+96]) for t < 32, a shuffle-down tree of distances 16..1, then
    bf16((x * inv) * gain) with inv = rsqrt(sum / 128 + eps).  Equal to rmsnorm() at this width.  The kernel's
    rsqrt.approx is not correctly rounded; `inv_ulps` moves inv by that many float32 steps so that a test can ask
    whether a result is explained by an approximation error of that size."""
    x = _f32(x)
    g = _f32(gain)
    sq = x * x
    t = (sq[..., 0:32] + sq[..., 64:96]) + (sq[..., 32:64] + sq[..., 96:128])
    d = 16
    while d > 0:
        t = t[..., :d] + t[..., d:2 * d]
        d //= 2
    arg = t[..., 0] / np.float32(128.0) + np.float32(eps)
    inv = (1.0 / np.sqrt(arg.astype(np.float64))).astype(np.float32)
    if inv_ulps:
        inv = (inv.view(np.int32) + np.int32(inv_ulps)).view(np.float32)
    return bf16((x * inv[..., None]) * g)


def head_norm_rope(x, gain, table, position: int, eps: float = 1e-6, inv_ulps: int = 0):
    """norm_rope / prepare_qk (src/kernels.rs:1292-1348, 1350-1443): head_norm, then rope.  x: [rows, heads, 128]."""
    return rope(head_norm(x, gain, eps, inv_ulps), table, position)


def head(x, w_bits):
    """The reference's bf16 output head, `head` (src/kernels.rs:2233-2257; `head_packed` :2259-2373 gives the same bits):
    logit[n] = bf16(sum_k x[k] * w[n, k]) with the float32 sum in the kernel's order -- lane L of a warp adds the
    products of columns L, L + 32, L + 64, ... in that order, then the 32 partial sums meet in a shuffle-down tree of
    distances 16, 8, 4, 2, 1.  x: [K] float32 (bf16 values), K a multiple of 32; w_bits: [N, K] bf16 bit patterns."""
    x = _f32(x).reshape(-1)
    w = from_bf16_bits(np.asarray(w_bits, np.uint16))
    n, k = w.shape
    assert k == x.size and k % 32 == 0
    prod = (w * x[None, :]).reshape(n, k // 32, 32)   # [row, step, lane]; one float32 rounding per product
    s = np.zeros((n, 32), np.float32)
    for step in range(k // 32):
        s = s + prod[:, step, :]
    d = 16
    while d > 0:
        s[:, :d] = s[:, :d] + s[:, d:2 * d]
        d //= 2
    return bf16(s[:, 0])


def attention(q, k_bits, v_bits, position: int):
    """src/kernels.rs:1490-1658.  q: [rows, q_heads, 128] float32 (bf16 values); k_bits, v_bits: [keys, kv_heads, 128]
    bf16 bit patterns with keys >= position + rows.  Row r sees keys 0 .. position + r.  Summation orders follow the
    kernel: score = sequential sum over the 128 channels, times 128^-0.5; exp(score - max) with the kernel's
    ex2.approx replaced by a correctly rounded exp (the one approximation in this restatement); the total as
    128 strided partial sums (key j goes to partial j % 128, in increasing j) folded by a tree of distances 64..1;
    one RN division per key; P.V as a sequential sum over the keys."""
    q = _f32(q)
    k = from_bf16_bits(np.asarray(k_bits, np.uint16))
    v = from_bf16_bits(np.asarray(v_bits, np.uint16))
    rows, heads, d = q.shape
    group = heads // k.shape[1]
    out = np.empty((rows, heads, d), np.float32)
    scale = np.float32(0.08838834764831845)
    for r in range(rows):
        end = position + r + 1
        for h in range(heads):
            kk = k[:end, h // group]          # [end, 128]
            vv = v[:end, h // group]
            s = np.zeros(end, np.float32)
            for c in range(d):
                s = s + q[r, h, c] * kk[:, c]
            s = s * scale
            e = np.exp((s + (-s.max())).astype(np.float64)).astype(np.float32)
            pad = np.zeros((end + 127) // 128 * 128, np.float32)
            pad[:end] = e
            part = np.zeros(128, np.float32)
            for chunk in pad.reshape(-1, 128):
                part = part + chunk
            n = 64
            while n > 0:
                part[:n] = part[:n] + part[n:2 * n]
                n //= 2
            p = e / part[0]
            acc = np.zeros(d, np.float32)
            for j in range(end):
                acc = acc + p[j] * vv[j]
            out[r, h] = bf16(acc)
    return out
