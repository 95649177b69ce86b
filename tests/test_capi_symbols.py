"""CPU-only checks of the C-ABI boundary: the built library loads without a GPU and exports exactly the
functions include/w8a8.h and include/qwen3_glue.h declare; the ctypes binding covers each of them.  No compute call is made."""
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def declared():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b((?:w8a8|qwen3)_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


@pytest.fixture(scope="module")
def lib():
    from inferrous_b200.build import build_library
    from inferrous_b200 import capi

    build_library()  # nvcc cross-compiles for sm_100a without a GPU
    return capi.load()


def test_header_declares_the_expected_surface(declared):
    for name in ("w8a8_init", "w8a8_weight_create", "w8a8_quantize", "w8a8_rmsnorm_quantize", "w8a8_swiglu_quantize",
                 "w8a8_linear", "w8a8_linear_grouped", "w8a8_linear_gate_up_swiglu", "w8a8_residual", "w8a8_device_status",
                 "qwen3_embedding", "qwen3_prepare_qk", "qwen3_attention"):
        assert name in declared


def test_library_exports_every_declared_symbol(lib, declared):
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/*.h but not exported by libw8a8.so"


def test_binding_covers_every_declared_symbol(declared):
    from inferrous_b200 import capi

    assert sorted(capi.SIGNATURES) == declared


def test_status_strings_and_version_need_no_gpu(lib):
    assert lib.w8a8_version().decode().count(".") == 2
    assert lib.w8a8_status_string(0) == b"ok"
    for code in range(1, 7):
        assert lib.w8a8_status_string(code) not in (b"ok", b"unknown status")
    assert lib.w8a8_status_string(99) == b"unknown status"


def test_argument_validation_needs_no_gpu(lib):
    # rejected before any CUDA call is made
    assert lib.w8a8_quantize(None, 0, 1, 128, 128, None, None, None) == 1
    assert lib.w8a8_linear(None, None, None, 1, None, None, None, 0, None) == 1
    assert lib.w8a8_weight_destroy(None) == 1
    assert lib.w8a8_init(-1) == 1
    # prefetch hints: a thread-local list of at most four ranges, cleared by (NULL, 0)
    assert lib.w8a8_prefetch_hint(None, 5) == 1
    import ctypes
    buf = ctypes.create_string_buffer(256)
    for _ in range(4):
        assert lib.w8a8_prefetch_hint(ctypes.addressof(buf), 256) == 0
    assert lib.w8a8_prefetch_hint(ctypes.addressof(buf), 256) == 3
    assert lib.w8a8_prefetch_hint(None, 0) == 0
    assert lib.w8a8_prefetch_hint(ctypes.addressof(buf), 256) == 0
    assert lib.w8a8_prefetch_hint(None, 0) == 0
    # the operators around the linear layers refuse to run before w8a8_init()
    assert lib.qwen3_embedding(None, None, 1, 4096, 10, None, 0, None) == 6
    assert lib.qwen3_attention(None, 0, 4096, 1, 32, 8, None, None, None, None, 4096, 4096, None, None) == 6
    # workspace sizing is host arithmetic
    offsets = (ctypes.c_size_t * 5)()
    total = lib.w8a8_workspace_bytes(129, 4096, 4096, 12288, offsets)
    assert list(offsets) == [0, 528384, 1056768, 2641920, 2642688] and total == 2643456
    assert lib.w8a8_workspace_bytes(0, 4096, 4096, 12288, None) == 0
    # the resident decode kernel's plan: nothing without w8a8_init(), no plan from a null handle
    out = ctypes.c_void_p()
    assert lib.qwen3_decode_plan_create(None, 1, 256, 4, 2, 512, 64, 1e-6, None, 0, ctypes.byref(out)) == 6
    assert lib.qwen3_decode_layers(None, None, None, None) == 1
    assert lib.qwen3_decode_plan_set_peers(None, None, None, 0, 1) == 1
    n = ctypes.c_int()
    assert lib.qwen3_decode_plan_trace(None, None, 0, ctypes.byref(n), ctypes.byref(n), ctypes.byref(n)) == 1
    assert lib.qwen3_decode_plan_destroy(None) == 0


def test_overlapping_operands_are_rejected_on_the_host(lib):
    """Inputs and outputs of a projection never share memory (docs/qwen3-8b-w8a8/safety.md:15).  The check runs on the
    host before any CUDA call, so it can be exercised here with made-up, suitably aligned addresses through the entry
    point that takes raw pointers; w8a8_linear / w8a8_linear_ex run the same check with the shapes of the weight handle."""
    base = 0x7000_0000_0000
    M, N, K = 17, 256, 512  # one token more than that entry point takes: a call that passes the check stops at the next one
    q, a, w, ws, y = base, base + (1 << 20), base + (2 << 20), base + (3 << 20), base + (4 << 20)
    call = lambda q=q, a=a, w=w, ws=ws, y=y, dtype=0: lib.w8a8_linear_no_alloc(q, a, w, ws, M, N, K, y, dtype, None)
    for kw, names in [(dict(y=q), b"output y overlaps input q"), (dict(y=w + N * K - 16), b"output y overlaps input w"),
                      (dict(y=ws), b"w_scale"), (dict(y=a - M * N * 2 + 16), b"a_scale"), (dict(y=q + M * K - 16), b"input q")]:
        assert call(**kw) == 1
        assert names in lib.w8a8_last_cuda_error()
    # adjacent ranges do not overlap: the call gets past this check and is refused by the next one (too many tokens,
    # W8A8_ERR_UNSUPPORTED), so nothing is ever launched with these addresses
    assert call(y=q + M * K) == 3
    assert call(y=w - M * N * 2) == 3
    # the f32 carrier doubles the output's extent
    assert call(y=w - M * N * 4 + 16, dtype=1) == 1 and call(y=w - M * N * 4, dtype=1) == 3


def test_product_does_not_import_the_oracle():
    """The oracle is test infrastructure: nothing under inferrous_b200/ may import, load or link it."""
    needles = ("import oracle", "from oracle", "w8a8_oracle", "oracle/", "oracle.py")
    for path in (ROOT / "inferrous_b200").rglob("*"):
        if path.suffix in {".py", ".cu", ".cuh", ".h"}:
            text = path.read_text()
            for n in needles:
                assert n not in text, f"{path} mentions {n!r}"
