"""Writes src/lib.rs of this crate from include/w8a8.h and include/qwen3_glue.h: one `extern "C"` declaration per
function the headers declare.  Run it after a header changes (`python crates/w8a8-sys/generate.py`);
tests/test_rust_binding.py fails when src/lib.rs is out of date."""
import re
from pathlib import Path
ROOT = Path(__file__).resolve().parents[2]
TYPES = {
 'int': 'c_int', 'float': 'f32', 'size_t': 'usize', 'int64_t': 'i64',
 'const void *': '*const c_void', 'void *': '*mut c_void', 'const int8_t *': '*const i8', 'int8_t *': '*mut i8',
 'const float *': '*const f32', 'float *': '*mut f32', 'const uint32_t *': '*const u32', 'uint32_t *': '*mut u32',
 'const uint16_t *': '*const u16', 'uint16_t *': '*mut u16', 'int32_t *': '*mut i32', 'int *': '*mut c_int',
 'w8a8_weight_t': '*mut W8a8Weight', 'w8a8_weight_t *': '*mut *mut W8a8Weight', 'const w8a8_weight_t *': '*const *mut W8a8Weight',
 'void *const *': '*const *mut c_void', 'uint32_t *const *': '*const *mut u32', 'const char *': '*const c_char',
 'int64_t *': '*mut i64', 'size_t *': '*mut usize',
 'const qwen3_layer_desc *': '*const Qwen3LayerDesc', 'qwen3_decode_plan_t': '*mut Qwen3DecodePlan',
 'qwen3_decode_plan_t *': '*mut *mut Qwen3DecodePlan', 'const struct w8a8_weight *': '*const W8a8Weight',
}
def struct_fields(h, name):
    """Fields of `typedef struct name {...} name;` as (field, rust type), one per declarator."""
    text = re.sub(r"/\*.*?\*/", "", (ROOT/h).read_text(), flags=re.S)
    body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), text, flags=re.S).group(1)
    out = []
    for decl in body.split(';'):
        decl = ' '.join(decl.split())
        if not decl:
            continue
        first, *rest = [d.strip() for d in decl.split(',')]
        m = re.match(r"(.*?)(\w+)$", first)
        ty = m.group(1).strip()
        out.append((m.group(2), TYPES[ty]))
        for more in rest:  # `*name`: the pointer belongs to the declarator
            out.append((more.lstrip('* '), TYPES[ty]))
    return out
def parse(h):
    text = re.sub(r"/\*.*?\*/", "", (ROOT/h).read_text(), flags=re.S)
    text = re.sub(r"#.*", "", text)
    out = []
    for m in re.finditer(r"\b(int|size_t|const char \*)\s*((?:w8a8|qwen3)_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        args = ' '.join(m.group(3).split())
        out.append((m.group(1).strip(), m.group(2), [] if args == 'void' else [a.strip() for a in args.split(',')]))
    return out
def arg(a):
    m = re.match(r"(.*?)(\w+)$", a)
    ty, name = m.group(1).strip(), m.group(2)
    name = {'type': 'ty', 'in': 'input'}.get(name, name).lower()
    return name, TYPES[ty]
lines = []
for h, title in [('include/w8a8.h', 'the W8A8 linear-layer path'), ('include/qwen3_glue.h', 'the operators around it')]:
    lines.append(f"    // ---- {h}: {title}")
    for ret, name, args in parse(h):
        rs = ', '.join(f"{n}: {t}" for n, t in map(arg, args))
        lines.append(f"    pub fn {name}({rs}) -> {TYPES.get(ret, 'c_int') if ret != 'int' else 'c_int'};")
body = '\n'.join(lines)
layer_fields = '\n'.join(f"    pub {n}: {t}," for n, t in struct_fields('include/qwen3_glue.h', 'qwen3_layer_desc'))
src = f'''//! Raw bindings to `libw8a8.so`, the sm_100a (B200) implementation of the W8A8 linear-layer path of
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

use std::os::raw::{{c_char, c_int, c_void}};

/// Opaque weight handle (`w8a8_weight_t`): device pointers, shape and TMA descriptors of one `[N, K]` int8 matrix.
#[repr(C)]
pub struct W8a8Weight {{
    _private: [u8; 0],
}}

/// Opaque plan of the resident decode kernel (`qwen3_decode_plan_t`).
#[repr(C)]
pub struct Qwen3DecodePlan {{
    _private: [u8; 0],
}}

/// One decoder layer as `qwen3_decode_plan_create` takes it (`qwen3_layer_desc`).
#[repr(C)]
pub struct Qwen3LayerDesc {{
{layer_fields}
}}

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
extern "C" {{
{body}
}}

/// `Err(status)` unless the call returned `W8A8_OK`; the text of a failing CUDA call is in `w8a8_last_cuda_error()`.
pub fn check(status: c_int) -> Result<(), c_int> {{
    if status == W8A8_OK {{
        Ok(())
    }} else {{
        Err(status)
    }}
}}
'''


def main():
    import sys

    target = ROOT / 'crates/w8a8-sys/src/lib.rs'
    if '--check' in sys.argv:
        sys.exit(0 if target.read_text() == src else 1)
    target.write_text(src)


if __name__ == '__main__':
    main()

