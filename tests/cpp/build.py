"""Compiles tests/cpp/conformance.cpp (host C++ only) against libw8a8.so and the CUDA runtime."""
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
OUT = HERE / "_build" / "conformance"


def build() -> Path:
    from inferrous_b200.build import build_library

    lib = build_library()
    OUT.parent.mkdir(exist_ok=True)
    src = HERE / "conformance.cpp"
    deps = [src, ROOT / "inferrous_b200" / "host" / "gpu_linear.hpp", ROOT / "include" / "w8a8.h", lib]
    if OUT.exists() and all(OUT.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return OUT
    cmd = ["g++", "-O2", "-std=c++17", "-ffp-contract=off", str(src), "-I/usr/local/cuda/include", "-L/usr/local/cuda/lib64",
           f"-L{lib.parent}", "-lw8a8", "-lcudart", f"-Wl,-rpath,{lib.parent}", "-Wl,-rpath,/usr/local/cuda/lib64", "-o", str(OUT)]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build())
