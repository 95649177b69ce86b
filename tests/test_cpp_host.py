"""The C++ host mirror (inferrous_b200/host/gpu_linear.hpp): it must compile against the C ABI on any box,
and on a GPU its conformance program (closed-form tests in the shape of the reference's conformance.rs) must pass."""
import subprocess

import pytest


def test_cpp_host_mirror_compiles_and_links():
    from tests.cpp.build import build

    exe = build()
    assert exe.exists()


@pytest.mark.gpu
def test_cpp_conformance_program():
    from tests.cpp.build import build

    r = subprocess.run([str(build())], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "conformance ok" in r.stdout
