"""GPU parity of the one-token projections whose quantizer runs in the projection kernel's prologue
(w8a8_quantize_linear, w8a8_quantize_linear_gate_up_swiglu): bit-identical to the quantizer entry point followed by
the projection entry point, and to the CPU restatement where that is exact.  All calls go through the C ABI."""
import numpy as np
import pytest

from oracle import oracle
from tests.util import bits, empty_act, synth_activations, synth_gamma, synth_weights, to_dev, to_host

pytestmark = pytest.mark.gpu

CARRIERS = ["bf16", "f32"]
TINY = np.float32(1e-8).view(np.uint32)


@pytest.fixture(scope="module")
def ops():
    from inferrous_b200 import ops as o

    o.init()
    return o


def matrix(ops, rng, N, K):
    w, ws = synth_weights(rng, N, K)
    return ops.Matrix(to_dev(w), to_dev(ws, "f32")), w, ws


@pytest.mark.parametrize("carrier", CARRIERS)
@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 4096), (4096, 12288), (640, 256), (33, 128)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_with_max_source_equals_quantize_then_linear(ops, carrier, N, K, with_residual):
    import torch

    rng = np.random.default_rng(N + K)
    mat, w, ws = matrix(ops, rng, N, K)
    x = synth_activations(rng, 1, K)
    res = oracle.bf16(rng.standard_normal((1, N)).astype(np.float32)) if with_residual else None
    m = max(np.float32(1e-8), np.abs(x).max())
    maxima = to_dev(np.array([np.float32(m).view(np.uint32)], np.uint32))
    xd = to_dev(x, carrier)
    # the two entry points one after the other
    q = torch.zeros((1, K), dtype=torch.int8, device="cuda")
    s = torch.zeros(1, dtype=torch.float32, device="cuda")
    ops.quantize_with_max(xd, maxima, q, s)
    y_ref, c_ref = empty_act((1, N), carrier), empty_act((1, N), carrier)
    if with_residual:
        ops.linear_residual(q, s, mat, y_ref, to_dev(res, carrier), c_ref)
    else:
        ops.linear_quantized(q, s, mat, y_ref)
    # one kernel
    y, c = empty_act((1, N), carrier), empty_act((1, N), carrier)
    q_out = torch.zeros_like(q)
    s_out = torch.zeros_like(s)
    reset = to_dev(np.array([5, 6, 7], np.uint32))
    ops.quantize_linear(xd, mat, y, maxima_in=maxima, residual_in=to_dev(res, carrier) if with_residual else None,
                        combined=c if with_residual else None, maxima_reset=reset, q_out=q_out, scale_out=s_out)
    assert torch.equal(q_out, q) and np.array_equal(bits(to_host(s_out)), bits(to_host(s)))
    assert np.array_equal(bits(to_host(y)), bits(to_host(y_ref)))
    if with_residual:
        assert np.array_equal(bits(to_host(c)), bits(to_host(c_ref)))
    assert np.all(to_host(reset).view(np.uint32) == TINY)
    # and the CPU restatement (exact for this source)
    eq, es = oracle.quantize(x)
    assert np.array_equal(to_host(q_out), eq) and np.array_equal(bits(to_host(s_out)), bits(es))
    expected = oracle.linear(eq, es, w, ws, residual_in=res)
    assert np.array_equal(bits(to_host(y)), bits(expected[0] if with_residual else expected))
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("carrier", CARRIERS)
@pytest.mark.parametrize("N,K", [(6144, 4096), (4096, 8192), (640, 256), (33, 128)])
def test_rmsnorm_source_equals_norm_quantize_then_linear(ops, carrier, N, K):
    import torch

    rng = np.random.default_rng(N * 3 + K)
    mat, w, ws = matrix(ops, rng, N, K)
    x = synth_activations(rng, 1, K)
    gamma = synth_gamma(rng, K)
    xd, gd = to_dev(x, carrier), to_dev(gamma, carrier)
    q = torch.zeros((1, K), dtype=torch.int8, device="cuda")
    s = torch.zeros(1, dtype=torch.float32, device="cuda")
    ops.norm_quantize(xd, gd, None, q, s, None)
    y_ref = empty_act((1, N), carrier)
    ops.linear_quantized(q, s, mat, y_ref)
    y = empty_act((1, N), carrier)
    q_out, s_out = torch.zeros_like(q), torch.zeros_like(s)
    ops.quantize_linear(xd, mat, y, gain=gd, q_out=q_out, scale_out=s_out)
    assert torch.equal(q_out, q) and np.array_equal(bits(to_host(s_out)), bits(to_host(s)))
    assert np.array_equal(bits(to_host(y)), bits(to_host(y_ref)))
    # given the codes the kernel produced, the projection is the CPU restatement's
    assert np.array_equal(bits(to_host(y)), bits(oracle.linear(to_host(q_out), to_host(s_out), w, ws)))
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("carrier", CARRIERS)
@pytest.mark.parametrize("source", ["rmsnorm", "with_max"])
@pytest.mark.parametrize("I,K", [(12288, 4096), (384, 256)])
def test_gate_up_swiglu_with_folded_quantizer(ops, carrier, source, I, K):
    import torch

    rng = np.random.default_rng(I + K)
    gate, _, _ = matrix(ops, rng, I, K)
    up, _, _ = matrix(ops, rng, I, K)
    x = synth_activations(rng, 1, K)
    xd = to_dev(x, carrier)
    q = torch.zeros((1, K), dtype=torch.int8, device="cuda")
    s = torch.zeros(1, dtype=torch.float32, device="cuda")
    kw = {}
    if source == "rmsnorm":
        gd = to_dev(synth_gamma(rng, K), carrier)
        ops.norm_quantize(xd, gd, None, q, s, None)
        kw["gain"] = gd
    else:
        maxima = to_dev(np.array([np.abs(x).max().view(np.uint32)], np.uint32))
        ops.quantize_with_max(xd, maxima, q, s)
        kw["maxima_in"] = maxima
    act_ref = empty_act((1, I), carrier)
    mx_ref = to_dev(np.array([TINY], np.uint32))
    ops.linear_swiglu(q, s, gate, up, None, None, act_ref, mx_ref)
    act = empty_act((1, I), carrier)
    mx = to_dev(np.array([TINY], np.uint32))
    ops.quantize_linear_swiglu(xd, gate, up, act, mx, **kw)
    assert np.array_equal(bits(to_host(act)), bits(to_host(act_ref)))
    assert torch.equal(mx, mx_ref)
    assert ops.device_status() == (0, 0)


def test_rejections(ops):
    import torch

    from inferrous_b200 import capi

    rng = np.random.default_rng(0)
    mat, _, _ = matrix(ops, rng, 128, 128)
    x = to_dev(synth_activations(rng, 1, 128), "bf16")
    y = empty_act((1, 128), "bf16")
    with pytest.raises(capi.W8A8Error) as e:  # neither a gain nor a maximum
        capi.check(capi.load().w8a8_quantize_linear(x.data_ptr(), 0, 1, None, 1e-6, None, mat.handle, None, y.data_ptr(), None,
                                                    None, 0, None, None, None), "w8a8_quantize_linear")
    assert e.value.status == 1
    big, _, _ = matrix(ops, rng, 16, 20480)
    xb = to_dev(synth_activations(rng, 1, 20480), "bf16")
    with pytest.raises(capi.W8A8Error) as e:  # the float32 copy of the row would not fit in shared memory
        ops.quantize_linear(xb, big, empty_act((1, 16), "bf16"), gain=xb)
    assert e.value.status == 3
