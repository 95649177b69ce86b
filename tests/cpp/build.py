"""Compiles the host C++ programs of tests/cpp/ (no device code) against libw8a8.so and the CUDA runtime."""
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
OUT_DIR = HERE / "_build"


def build(program: str = "conformance") -> Path:
    from inferrous_b200.build import build_library

    lib = build_library()
    OUT_DIR.mkdir(exist_ok=True)
    out = OUT_DIR / program
    src = HERE / f"{program}.cpp"
    deps = [src, lib, *sorted((ROOT / "inferrous_b200" / "host").glob("*.hpp")), *sorted((ROOT / "include").glob("*.h"))]
    if out.exists() and all(out.stat().st_mtime >= d.stat().st_mtime for d in deps):
        return out
    cmd = ["g++", "-O2", "-std=c++17", "-ffp-contract=off", str(src), "-I/usr/local/cuda/include", "-L/usr/local/cuda/lib64",
           f"-L{lib.parent}", "-lw8a8", "-lcudart", f"-Wl,-rpath,{lib.parent}", "-Wl,-rpath,/usr/local/cuda/lib64", "-o", str(out)]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    print(build("conformance"), build("generate"))
