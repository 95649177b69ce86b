"""The allocation-free projection entry point (w8a8_linear_no_alloc) against the regular one.

Some callers of this library cannot allocate device memory: a plug-in that is given buffers and a
stream by its host application, code that runs after the process has closed its memory pool, or code
inside a stream capture owned by someone else.  For them the library keeps the scratch of its stream-K
kernel in a fixed device array.  This test calls that entry point through the C ABI twice in a row (the
array is shared by all calls and keeps its contents, so the second call checks that the first one's
leftovers do no harm) and compares bit for bit with w8a8_linear.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.  It passes alone in a fresh process too: the new entry point is called BEFORE the
library's regular set-up (w8a8_init), which it must not need."""
import numpy as np
import pytest

from tests.util import bits, empty_act, to_dev, to_host

pytestmark = pytest.mark.gpu


def make_case(seed, M, K, N):
    rng = np.random.default_rng(seed)
    q = rng.integers(-127, 128, (M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    q[0] = 127
    w[0] = 127
    w[1] = -127
    asc = (rng.random(M, dtype=np.float32) / 64).astype(np.float32)
    ws = (rng.random(N, dtype=np.float32) / 64).astype(np.float32)
    return q, w, asc, ws


def test_no_alloc_matches_regular_entry_point_twice_in_a_row():
    import torch
    from inferrous_b200 import capi, ops

    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    cases = [make_case(1, 16, 4096, 4096), make_case(2, 5, 4096, 4096)]  # K blocks of a tile are split over CTAs
    dev = []
    for q, w, asc, ws in cases:
        dev.append((to_dev(q), to_dev(asc, "f32"), to_dev(w), to_dev(ws, "f32")))
    # two calls in a row through the allocation-free entry point, before any regular set-up
    outs = []
    for (qd, ad, wd, wsd), (q, w, _, _) in zip(dev, cases):
        y = empty_act((q.shape[0], w.shape[0]), "bf16")
        ops.linear_no_alloc(qd, ad, wd, wsd, y)
        outs.append(y)
    torch.cuda.synchronize()
    # the regular entry point (needs w8a8_init and a weight handle, both of which allocate)
    ops.init()
    for (qd, ad, wd, wsd), (q, w, _, _), y in zip(dev, cases, outs):
        mat = ops.Matrix(wd, wsd)
        ref = empty_act((q.shape[0], w.shape[0]), "bf16")
        ops.linear_quantized(qd, ad, mat, ref)
        assert np.array_equal(bits(to_host(y)), bits(to_host(ref)))
        ref2 = empty_act((q.shape[0], w.shape[0]), "bf16")
        ops.linear_quantized(qd, ad, mat, ref2, capi.VARIANT_NAIVE)
        assert np.array_equal(bits(to_host(y)), bits(to_host(ref2)))
    # f32 carrier, and once more after the regular path has run
    qd, ad, wd, wsd = dev[0]
    y32 = empty_act((16, 4096), "f32")
    ops.linear_no_alloc(qd, ad, wd, wsd, y32)
    assert np.array_equal(bits(to_host(y32)), bits(to_host(outs[0])))


def test_no_alloc_rejects_what_its_fixed_scratch_cannot_hold():
    import torch
    from inferrous_b200 import capi

    lib = capi.load()
    q = torch.zeros((17, 128), dtype=torch.int8, device="cuda")
    a = torch.ones((17,), dtype=torch.float32, device="cuda")
    w = torch.zeros((128, 128), dtype=torch.int8, device="cuda")
    ws = torch.ones((128,), dtype=torch.float32, device="cuda")
    y = torch.zeros((17, 128), dtype=torch.bfloat16, device="cuda")
    st = lib.w8a8_linear_no_alloc(q.data_ptr(), a.data_ptr(), w.data_ptr(), ws.data_ptr(), 17, 128, 128, y.data_ptr(), 0, None)
    assert st == 3
    assert b"16 tokens" in lib.w8a8_last_cuda_error()
    assert lib.w8a8_linear_no_alloc(None, a.data_ptr(), w.data_ptr(), ws.data_ptr(), 1, 128, 128, y.data_ptr(), 0, None) == 1


@pytest.mark.parametrize("M,K,N", [
    (3, 4096, 200),    # a partial last tile of 128 channels
    (16, 4096, 64),    # fewer channels than one tile
    (7, 128, 384),     # one K block: one block per stage, no tile is split
    (2, 384, 1000),    # three K blocks: one block per stage
    (1, 12288, 4096),  # one token, the longest K of the model
    (9, 512, 128),     # a single tile whose four K blocks make one unit: one CTA, nothing split
])
def test_no_alloc_small_and_ragged_shapes(M, K, N):
    """Partial tiles, every stage width, one token, split and unsplit tiles: bit for bit the one-thread-per-output kernel.
    Afterwards no wait is on record: w8a8_device_status also reads the status words inside the fixed array."""
    from inferrous_b200 import capi, ops

    q, w, asc, ws = make_case(M * 1000 + N, M, K, N)
    qd, ad, wd, wsd = to_dev(q), to_dev(asc, "f32"), to_dev(w), to_dev(ws, "f32")
    for _ in range(2):
        y = empty_act((M, N), "bf16")
        ops.linear_no_alloc(qd, ad, wd, wsd, y)
        ops.init()
        ref = empty_act((M, N), "bf16")
        ops.linear_quantized(qd, ad, ops.Matrix(wd, wsd), ref, capi.VARIANT_NAIVE)
        assert np.array_equal(bits(to_host(y)), bits(to_host(ref)))
    assert ops.device_status() == (0, 0)
