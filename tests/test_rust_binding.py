"""The Rust FFI crate (crates/w8a8-sys) against the C headers.  No Rust toolchain exists where this library is built, so
the crate cannot be compiled here; what can be checked is that it declares exactly the functions the headers declare,
with the same number of arguments and the matching Rust type for every C type, and the same constants."""
import re
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
LIB_RS = ROOT / "crates" / "w8a8-sys" / "src" / "lib.rs"

C_TO_RUST = {
    "int": "c_int", "float": "f32", "size_t": "usize", "int64_t": "i64", "const void *": "*const c_void", "void *": "*mut c_void",
    "const int8_t *": "*const i8", "int8_t *": "*mut i8", "const float *": "*const f32", "float *": "*mut f32",
    "const uint32_t *": "*const u32", "uint32_t *": "*mut u32", "const uint16_t *": "*const u16", "uint16_t *": "*mut u16",
    "int32_t *": "*mut i32", "int *": "*mut c_int", "w8a8_weight_t": "*mut W8a8Weight", "w8a8_weight_t *": "*mut *mut W8a8Weight",
    "const w8a8_weight_t *": "*const *mut W8a8Weight", "void *const *": "*const *mut c_void", "uint32_t *const *": "*const *mut u32",
    "const char *": "*const c_char", "int64_t *": "*mut i64", "size_t *": "*mut usize", "const qwen3_layer_desc *": "*const Qwen3LayerDesc", "qwen3_decode_plan_t": "*mut Qwen3DecodePlan",
    "qwen3_decode_plan_t *": "*mut *mut Qwen3DecodePlan", "const struct w8a8_weight *": "*const W8a8Weight",
}


def header_functions():
    out = {}
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        text = re.sub(r"#.*", "", text)
        for m in re.finditer(r"\b(int|size_t|const char \*)\s*((?:w8a8|qwen3)_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
            args = " ".join(m.group(3).split())
            types = [] if args == "void" else [re.match(r"(.*?)\w+$", a.strip()).group(1).strip() for a in args.split(",")]
            out[m.group(2)] = (m.group(1).strip(), types)
    return out


def rust_functions():
    text = LIB_RS.read_text()
    block = text[text.index('extern "C" {'):]
    out = {}
    for m in re.finditer(r"pub fn (\w+)\((.*?)\) -> ([^;]+);", block):
        args = [a.split(":", 1)[1].strip() for a in m.group(2).split(",") if a.strip()]
        out[m.group(1)] = (m.group(3).strip(), args)
    return out


def test_every_header_function_is_declared_with_matching_types():
    c, rust = header_functions(), rust_functions()
    assert len(c) >= 38
    assert sorted(c) == sorted(rust)
    for name, (ret, types) in c.items():
        rret, rtypes = rust[name]
        assert rret == C_TO_RUST[ret], name
        assert rtypes == [C_TO_RUST[t] for t in types], name


def test_layer_struct_matches_the_header():
    header = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / "qwen3_glue.h").read_text(), flags=re.S)
    body = re.search(r"typedef struct qwen3_layer_desc \{(.*?)\} qwen3_layer_desc;", header, flags=re.S).group(1)
    fields = []
    for decl in body.split(";"):
        decl = " ".join(decl.split())
        if decl:
            first, *rest = [d.strip() for d in decl.split(",")]
            ty, name = re.match(r"(.*?)(\w+)$", first).groups()
            fields += [(name, C_TO_RUST[ty.strip()])] + [(more.lstrip("* "), C_TO_RUST[ty.strip()]) for more in rest]
    rust = LIB_RS.read_text()
    block = re.search(r"pub struct Qwen3LayerDesc \{(.*?)\}", rust, flags=re.S).group(1)
    assert re.findall(r"pub (\w+): ([^,]+),", block) == fields and len(fields) == 11


def test_constants_match_the_header():
    header = (ROOT / "include" / "w8a8.h").read_text()
    rust = LIB_RS.read_text()
    values = dict(re.findall(r"\b(W8A8_[A-Z0-9_]+)\s*=\s*(\d+)", re.sub(r"/\*.*?\*/", "", header, flags=re.S)))
    values.update(re.findall(r"#define (W8A8_SOURCE_[A-Z_]+) (\d+)", header))
    declared = dict(re.findall(r"pub const (W8A8_[A-Z0-9_]+): c_int = (\d+);", rust))
    assert declared == values


def test_generated_file_is_up_to_date():
    r = subprocess.run([sys.executable, str(ROOT / "crates" / "w8a8-sys" / "generate.py"), "--check"])
    assert r.returncode == 0, "crates/w8a8-sys/src/lib.rs is stale: run python crates/w8a8-sys/generate.py"
