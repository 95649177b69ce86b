"""Builds libw8a8.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

No torch, no JIT cache: plain `nvcc -shared`, one object per .cu file, statically linked
CUDA runtime, the driver entry point for tensor-map encoding resolved at run time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libw8a8.so"
OBJ_DIR = PKG / "lib" / "obj"
SOURCES = ["capi.cu", "quantize.cu", "naive.cu", "gemv.cu", "gemm_tcgen05.cu", "gemm_tcgen05_pair.cu", "gemm_skinny.cu", "gemm_cluster.cu", "tp_allreduce.cu", "forward_glue.cu", "batched_decode.cu", "head_bf16.cu", "decode_layers.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "--fmad=false",            # the reference builds with FMA contraction off (tools/cuda.sh:21)
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "w8a8.h", PKG.parent / "include" / "qwen3_glue.h", Path(__file__)]
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    cc = nvcc()
    jobs = []
    for src in SOURCES:
        obj = OBJ_DIR / (src + ".o")
        if force or _stale(obj, [CSRC / src] + headers):
            cmd = [cc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if ptxas_info else []), "-c", str(CSRC / src), "-o", str(obj)]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        for out in ex.map(run, jobs):
            if (verbose or ptxas_info) and out:
                print(out, file=sys.stderr)
    objs = [str(OBJ_DIR / (s + ".o")) for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        run([cc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *objs])
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
