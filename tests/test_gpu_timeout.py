"""A bounded device-side wait that runs out is reported, not hung on: the one-shot tensor-parallel all-reduce
(w8a8_tp_allreduce) is called as rank 0 of a group of two whose second rank never pushes -- both "peers" are buffers on
this GPU, and nothing ever sets the flag that rank 0 waits for.  After its time limit (about two seconds) the kernel
records the wait's code and returns; w8a8_device_status reports W8A8_ERR_DEVICE_TIMEOUT once, returns the library's shared
scratch to zero, and the calls that follow are right again.  No kernel is trapped, faulted or left spinning."""
import ctypes as C
import time

import numpy as np
import pytest

from tests.util import bits, empty_act, to_dev, to_host

pytestmark = pytest.mark.gpu


def test_expired_peer_wait_is_reported_and_the_library_stays_usable():
    import torch

    from inferrous_b200 import capi, ops

    ops.init()
    lib = capi.load()
    assert ops.device_status() == (0, 0)
    tp, n = 2, 4096
    partial = torch.randn(n, device="cuda").to(torch.bfloat16)
    out = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    bufs = [torch.zeros(2 * tp * n, dtype=torch.bfloat16, device="cuda") for _ in range(tp)]     # [2 halves][tp slots][n]
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(tp)]
    seq = torch.zeros(4, dtype=torch.int32, device="cuda")
    buf_ptrs = (C.c_void_p * tp)(*[b.data_ptr() for b in bufs])
    flag_ptrs = (C.c_void_p * tp)(*[f.data_ptr() for f in flags])
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    start = time.perf_counter()
    st = lib.w8a8_tp_allreduce(C.c_void_p(partial.data_ptr()), C.c_void_p(out.data_ptr()), n, capi.BF16, buf_ptrs, flag_ptrs,
                               C.c_void_p(seq.data_ptr()), 0, tp, n, stream)
    assert st == 0  # the launch itself succeeds; the wait runs out on the device
    torch.cuda.synchronize()
    waited = time.perf_counter() - start
    assert 1.0 < waited < 10.0, waited
    status, detail = ops.device_status()
    assert status == 5 and detail >> 24 == 5 and (detail & 0xFFFFFF) == 1  # WAIT_PEER, waiting for rank 1
    assert ops.device_status() == (0, 0)  # reading cleared it
    # rank 0's own push did arrive (slot 0 of both buffers), rank 1's slot is untouched
    assert torch.equal(bufs[0][:n], partial) and torch.equal(bufs[1][:n], partial) and not bufs[0][n:2 * n].any()
    # the library is still right: a stream-K projection (whose scratch the status call has just returned to zero) and a
    # streaming one, against the one-thread-per-output kernel
    rng = np.random.default_rng(7)
    for M, K, N, variant in [(16, 4096, 1024, capi.VARIANT_GEMM_SKINNY), (3, 1024, 512, capi.VARIANT_AUTO)]:
        q = rng.integers(-127, 128, (M, K), dtype=np.int8)
        w = rng.integers(-127, 128, (N, K), dtype=np.int8)
        asc = (rng.random(M, dtype=np.float32) / 64).astype(np.float32)
        ws = (rng.random(N, dtype=np.float32) / 64).astype(np.float32)
        mat = ops.Matrix(to_dev(w), to_dev(ws, "f32"))
        y, ref = empty_act((M, N), "bf16"), empty_act((M, N), "bf16")
        ops.linear_quantized(to_dev(q), to_dev(asc, "f32"), mat, y, variant)
        ops.linear_quantized(to_dev(q), to_dev(asc, "f32"), mat, ref, capi.VARIANT_NAIVE)
        assert np.array_equal(bits(to_host(y)), bits(to_host(ref)))
    assert ops.device_status() == (0, 0)
