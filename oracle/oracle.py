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
