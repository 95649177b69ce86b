"""ctypes binding of include/w8a8.h and include/qwen3_glue.h.  Every symbol the headers declare is bound here."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libw8a8.so"

OK = 0
BF16, F32 = 0, 1
SOURCE_WITH_MAX, SOURCE_RMSNORM = 1, 2
VARIANT_AUTO, VARIANT_NAIVE, VARIANT_GEMV_DP4A, VARIANT_GEMV_MMA, VARIANT_GEMM_TCGEN05, VARIANT_GEMM_SKINNY = range(6)
VARIANT_GEMM_TCGEN05_PAIR = 8
VARIANT_GEMM_CLUSTER = 9  # 6 and 7 were kernels that lost to the others everywhere and are gone

_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/w8a8.h one to one
SIGNATURES = {
    "w8a8_init": (_i, [_i]),
    "w8a8_version": (C.c_char_p, []),
    "w8a8_status_string": (C.c_char_p, [_i]),
    "w8a8_last_cuda_error": (C.c_char_p, []),
    "w8a8_set_programmatic_launch": (_i, [_i]),
    "w8a8_prefetch_hint": (_i, [_vp, _sz]),
    "w8a8_device_status": (_i, [_vp, C.POINTER(C.c_uint32)]),
    "w8a8_workspace_bytes": (_sz, [_i, _i, _i, _i, C.POINTER(_sz)]),
    "w8a8_weight_create": (_i, [_vp, _vp, _i, _i, C.POINTER(_vp)]),
    "w8a8_weight_destroy": (_i, [_vp]),
    "w8a8_weight_shape": (_i, [_vp, C.POINTER(_i), C.POINTER(_i)]),
    "w8a8_quantize": (_i, [_vp, _i, _i, _i, _i64, _vp, _vp, _vp]),
    "w8a8_quantize_with_max": (_i, [_vp, _i, _vp, _i, _i, _i64, _vp, _vp, _vp]),
    "w8a8_rmsnorm_quantize": (_i, [_vp, _vp, _i, _f, _i, _i, _i64, _vp, _vp, _vp, _vp, _vp]),
    "w8a8_swiglu": (_i, [_vp, _vp, _i, _i, _i, _i64, _vp, _vp, _vp]),
    "w8a8_swiglu_quantize": (_i, [_vp, _vp, _i, _i, _i, _i64, _vp, _vp, _vp, _vp]),
    "w8a8_residual": (_i, [_vp, _vp, _i, _sz, _vp, _vp]),
    "w8a8_linear": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp]),
    "w8a8_linear_ex": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "w8a8_linear_grouped": (_i, [_vp, _vp, C.POINTER(_vp), _i, _i, C.POINTER(_vp), _i, _vp]),
    "w8a8_linear_gate_up_swiglu": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp]),
    "w8a8_quantize_linear": (_i, [_vp, _i, _i, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp]),
    "w8a8_quantize_linear_gate_up_swiglu": (_i, [_vp, _i, _i, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "w8a8_linear_no_alloc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "w8a8_linear_argmax": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp]),
    "w8a8_linear_allreduce": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _i, C.POINTER(_vp), _vp, _i, _i, _sz, _vp]),
    "w8a8_tp_allreduce": (_i, [_vp, _vp, _sz, _i, C.POINTER(_vp), C.POINTER(_vp), _vp, _i, _i, _sz, _vp]),
    "w8a8_linear_acc_i32": (_i, [_vp, _vp, _i, _vp, _i, _vp]),
    "w8a8_rounding_probe": (_i, [_vp, _vp, _sz, _vp]),
    # include/qwen3_glue.h
    "qwen3_embedding": (_i, [_vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "qwen3_prepare_qk": (_i, [_vp, _i, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "qwen3_prepare_qk_batched": (_i, [_vp, _i, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _vp]),
    "qwen3_attention_batched_workspace": (_sz, [_i, _i, _i]),
    "qwen3_attention_batched": (_i, [_vp, _i, _i64, _i, _i, _i, _vp, _vp, _i64, _vp, _vp, _i64, _i, _vp, _vp, _sz, _vp]),
    "qwen3_head_bf16": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp]),
    "qwen3_select_token": (_i, [_vp, _i, _i, _i, _i64, _vp, _vp, _vp]),
    "qwen3_merge_candidates": (_i, [_vp, _i, _i, _i, _vp, _vp]),
    "qwen3_decode_plan_create": (_i, [_vp, _i, _i, _i, _i, _i, _i, _f, _vp, _i, C.POINTER(_vp)]),
    "qwen3_decode_plan_destroy": (_i, [_vp]),
    "qwen3_decode_layers": (_i, [_vp, _vp, _vp, _vp]),
    "qwen3_decode_plan_set_peers": (_i, [_vp, C.POINTER(_vp), _vp, _i, _i]),
    "qwen3_decode_plan_trace": (_i, [_vp, _vp, _sz, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "qwen3_attention_use_tensor_cores": (_i, [_i]),
    "qwen3_attention_quantize": (_i, [_vp, _i, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _i64, _i, _vp, _vp, _vp]),
    "qwen3_attention": (_i, [_vp, _i, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _i64, _i, _vp, _vp]),
}


class LayerDesc(C.Structure):
    """qwen3_layer_desc (include/qwen3_glue.h)."""
    _fields_ = [("norm1", _vp), ("qkv", _vp), ("q_gain", _vp), ("k_gain", _vp), ("o", _vp), ("norm2", _vp), ("gate", _vp),
                ("up", _vp), ("down", _vp), ("k_cache", _vp), ("v_cache", _vp)]


class W8A8Error(RuntimeError):
    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        super().__init__(f"{where}: status {status} ({detail})")


_lib = None


def load() -> C.CDLL:
    """Load libw8a8.so.  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m inferrous_b200.build` (needs nvcc). "
                "There is no CPU or PyTorch fallback.")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, where: str) -> None:
    if status != OK:
        lib = load()
        msg = lib.w8a8_status_string(status).decode()
        if status == 4:
            msg += ": " + lib.w8a8_last_cuda_error().decode()
        raise W8A8Error(status, where, msg)
