"""GPU parity of the activation quantizers against the CPU oracle and the reference's fixtures.
Mirrors the `quantize` / `norm` / `swiglu` / `residual` arms of independent_operators
(src/conformance.rs:75-202) and integer_rounding_boundaries (:841-871).  All calls go through
the C ABI (inferrous_b200.ops -> libw8a8.so)."""
import numpy as np
import pytest

from oracle import oracle
from tests.test_oracle_golden import rounding_expected, rounding_inputs
from tests.util import bits, empty_act, gate, synth_activations, synth_gamma, to_dev, to_host

pytestmark = pytest.mark.gpu

CARRIERS = ["bf16", "f32"]


@pytest.fixture(scope="module")
def ops():
    import torch
    from inferrous_b200 import ops as o

    assert torch.cuda.is_available()
    o.init()
    return o


def run_quantize(ops, x, carrier):
    import torch

    M, K = x.shape
    q = torch.full((M, K), 99, dtype=torch.int8, device="cuda")
    s = torch.full((M,), -1.0, dtype=torch.float32, device="cuda")
    ops.quantize(to_dev(x, carrier), q, s)
    return to_host(q), to_host(s)


@pytest.mark.parametrize("carrier", CARRIERS)
def test_quantize_fixtures_exact(ops, fixtures, carrier):
    for c in fixtures.cases("quantize"):
        x = fixtures.tensor(c, "x")
        q, s = run_quantize(ops, x, carrier)
        assert np.array_equal(q, fixtures.tensor(c, "q")), c["name"]
        assert np.array_equal(bits(s), bits(fixtures.tensor(c, "scale").reshape(-1))), c["name"]


@pytest.mark.parametrize("carrier", CARRIERS)
def test_quantize_with_max_fixtures_exact(ops, fixtures, carrier):
    import torch

    for c in fixtures.cases("quantize"):
        x = fixtures.tensor(c, "x")
        M, K = x.shape
        m = np.maximum(np.abs(x).max(-1), np.float32(1e-8)).astype(np.float32)
        q = torch.zeros((M, K), dtype=torch.int8, device="cuda")
        s = torch.zeros((M,), dtype=torch.float32, device="cuda")
        ops.quantize_with_max(to_dev(x, carrier), to_dev(m.view(np.uint32)), q, s)
        assert np.array_equal(to_host(q), fixtures.tensor(c, "q"))
        assert np.array_equal(bits(to_host(s)), bits(fixtures.tensor(c, "scale").reshape(-1)))


@pytest.mark.parametrize("carrier", CARRIERS)
@pytest.mark.parametrize("M,K", [(1, 4096), (4, 12288), (17, 4096), (129, 12288), (512, 4096), (3, 128), (5, 24576)])
def test_quantize_synthetic_exact(ops, carrier, M, K):
    rng = np.random.default_rng(824 + M + K)
    x = synth_activations(rng, M, K)
    x[0, :8] = [127.0, -127.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5]
    if M > 2:
        x[2] = 0.0  # empty row: scale floor, zero codes
    q, s = run_quantize(ops, x, carrier)
    eq, es = oracle.quantize(x)
    assert np.array_equal(q, eq)
    assert np.array_equal(bits(s), bits(es))


def test_quantize_strided_rows_and_nan(ops):
    """Rows taken out of a wider buffer (ld > K), and NaN handling: NaN is ignored by the row maximum
    and converts to code 0 (src/kernels.rs:25-34,436)."""
    import torch

    rng = np.random.default_rng(7)
    wide = synth_activations(rng, 6, 8192)
    wide[1, 5] = np.nan
    wide[4, 4095] = np.inf
    xd = to_dev(wide, "f32")[:, :4096]
    assert xd.stride(0) == 8192
    q = torch.zeros((6, 4096), dtype=torch.int8, device="cuda")
    s = torch.zeros((6,), dtype=torch.float32, device="cuda")
    ops.quantize(xd, q, s)
    eq, es = oracle.quantize(wide[:, :4096].copy())
    assert np.array_equal(to_host(q), eq)
    assert np.array_equal(bits(to_host(s)), bits(es))
    assert to_host(q)[1, 5] == 0


def test_integer_rounding_boundaries(ops):
    import torch

    x = rounding_inputs()
    out = torch.zeros(x.size, dtype=torch.int8, device="cuda")
    ops.rounding_probe(to_dev(x, "f32"), out)
    assert np.array_equal(to_host(out), rounding_expected(x))


@pytest.mark.parametrize("carrier", CARRIERS)
def test_norm_quantize_fixtures(ops, fixtures, carrier):
    """Fused norm+quantize: the bf16 norm row passes the reference's numeric gate against the fixture,
    and codes/scales are bit-exact given that row (the structure of src/conformance.rs:161-202)."""
    import torch

    for c in fixtures.cases("norm"):
        x, gain = fixtures.tensor(c, "x"), fixtures.tensor(c, "gain")
        M, K = x.shape
        y = empty_act((M, K), carrier)
        q = torch.zeros((M, K), dtype=torch.int8, device="cuda")
        s = torch.zeros((M,), dtype=torch.float32, device="cuda")
        mx = torch.zeros((M,), dtype=torch.int32, device="cuda")
        ops.norm_quantize(to_dev(x, carrier), to_dev(gain, carrier), y, q, s, mx)
        yh = to_host(y)
        gate(yh, fixtures.tensor(c, "out"))
        eq, es = oracle.quantize(yh)
        assert np.array_equal(to_host(q), eq)
        assert np.array_equal(bits(to_host(s)), bits(es))
        assert np.all(to_host(mx).view(np.uint32) == np.float32(1e-8).view(np.uint32))
        # without the optional outputs the codes are the same
        q2 = torch.zeros_like(q)
        s2 = torch.zeros_like(s)
        ops.norm_quantize(to_dev(x, carrier), to_dev(gain, carrier), None, q2, s2, None)
        assert torch.equal(q, q2) and torch.equal(s, s2)


@pytest.mark.parametrize("M,K", [(1, 4096), (16, 4096), (129, 4096), (512, 4096), (4096, 4096)])
def test_norm_quantize_synthetic(ops, M, K):
    import torch

    rng = np.random.default_rng(M)
    x = synth_activations(rng, M, K)
    gamma = synth_gamma(rng, K)
    y = empty_act((M, K), "bf16")
    q = torch.zeros((M, K), dtype=torch.int8, device="cuda")
    s = torch.zeros((M,), dtype=torch.float32, device="cuda")
    ops.norm_quantize(to_dev(x, "bf16"), to_dev(gamma, "bf16"), y, q, s, None)
    yh = to_host(y)
    ref = oracle.rmsnorm(x, gamma)
    gate(yh, ref)
    # how often the hardware rsqrt.approx path lands on the same bf16 as the correctly rounded oracle
    same = float((bits(yh) == bits(ref)).mean())
    assert same > 0.95, same
    eq, es = oracle.quantize(yh)
    assert np.array_equal(to_host(q), eq)
    assert np.array_equal(bits(to_host(s)), bits(es))


@pytest.mark.parametrize("carrier", CARRIERS)
def test_swiglu_fixture_and_maxima(ops, fixtures, carrier):
    import torch

    (c,) = fixtures.cases("swiglu")
    g, u = fixtures.tensor(c, "gate").reshape(1, -1), fixtures.tensor(c, "up").reshape(1, -1)
    act = empty_act(g.shape, carrier)
    mx = to_dev(np.array([np.float32(1e-8).view(np.uint32)], dtype=np.uint32))
    ops.swiglu(to_dev(g, carrier), to_dev(u, carrier), act, mx)
    a = to_host(act)
    gate(a, fixtures.tensor(c, "out").reshape(1, -1))
    expect_max = max(np.float32(1e-8), np.abs(a[np.isfinite(a)]).max())
    assert to_host(mx).view(np.uint32)[0] == np.float32(expect_max).view(np.uint32)


@pytest.mark.parametrize("carrier", CARRIERS)
@pytest.mark.parametrize("M,I", [(1, 12288), (5, 12288), (129, 12288), (3, 128), (512, 12288), (4096, 12288)])
def test_swiglu_quantize_equals_separate(ops, carrier, M, I):
    """Fused SwiGLU+quantize == `swiglu` then `quantize` bit for bit; act within the numeric gate of the oracle;
    also with gate|up interleaved as one [M,2I] buffer."""
    import torch

    rng = np.random.default_rng(I + M)
    gu = oracle.bf16(rng.standard_normal((M, 2 * I), dtype=np.float32) * 3.0)
    gud = to_dev(gu, carrier)
    gd, ud = gud[:, :I], gud[:, I:]
    act_sep = empty_act((M, I), carrier)
    ops.swiglu(gd, ud, act_sep, None)
    q_sep = torch.zeros((M, I), dtype=torch.int8, device="cuda")
    s_sep = torch.zeros((M,), dtype=torch.float32, device="cuda")
    ops.quantize(act_sep, q_sep, s_sep)
    act = empty_act((M, I), carrier)
    q = torch.zeros_like(q_sep)
    s = torch.zeros_like(s_sep)
    ops.swiglu_quantize(gd, ud, q, s, act)
    assert torch.equal(act.view(torch.int16 if carrier == "bf16" else torch.int32),
                       act_sep.view(torch.int16 if carrier == "bf16" else torch.int32))
    assert torch.equal(q, q_sep) and torch.equal(s, s_sep)
    a = to_host(act)
    ref, _ = oracle.swiglu(gu[:, :I], gu[:, I:])
    gate(a, ref)
    eq, es = oracle.quantize(a)
    assert np.array_equal(to_host(q), eq) and np.array_equal(bits(to_host(s)), bits(es))
    # maxima from `swiglu` feed quantize_with_max (the decode route, src/gpu.rs:377-390)
    mx = to_dev(np.full(M, np.float32(1e-8).view(np.uint32), dtype=np.uint32))
    ops.swiglu(gd, ud, act_sep, mx)
    q3 = torch.zeros_like(q)
    s3 = torch.zeros_like(s)
    ops.quantize_with_max(act_sep, mx, q3, s3)
    assert torch.equal(q3, q) and torch.equal(s3, s)


@pytest.mark.parametrize("carrier", CARRIERS)
def test_residual_fixture_exact(ops, fixtures, carrier):
    (c,) = fixtures.cases("residual")
    a, b = fixtures.tensor(c, "a"), fixtures.tensor(c, "b")
    out = empty_act(a.shape, carrier)
    ops.residual(to_dev(a, carrier), to_dev(b, carrier), out)
    assert np.array_equal(bits(to_host(out)), bits(fixtures.tensor(c, "out")))


def test_bad_arguments_are_rejected(ops):
    """The C ABI returns error codes (no traps, no exceptions across the boundary)."""
    import torch
    from inferrous_b200 import capi

    x = torch.zeros((2, 100), dtype=torch.bfloat16, device="cuda")  # K not a multiple of 128
    q = torch.zeros((2, 100), dtype=torch.int8, device="cuda")
    s = torch.zeros((2,), dtype=torch.float32, device="cuda")
    with pytest.raises(capi.W8A8Error) as e:
        ops.quantize(x, q, s)
    assert e.value.status == 2
    lib = capi.load()
    assert lib.w8a8_quantize(None, 0, 1, 128, 128, None, None, None) == 1
    assert lib.w8a8_quantize(x.data_ptr(), 7, 2, 128, 128, q.data_ptr(), s.data_ptr(), None) == 1


@pytest.mark.parametrize("carrier", CARRIERS)
def test_quantize_near_rounding_ties_exact(ops, carrier):
    """Rows whose quotients x/scale sit on, or a few ulps beside, every half-integer k+0.5: the kernel's multiply
    with exact-division fallback must give the codes of a true IEEE division (src/kernels.rs:448)."""
    rng = np.random.default_rng(5)
    rows = []
    for amax in (127.0, 100.25, 3.0, 0.0123, 77.7, 1e-3, 250.0):
        amax = oracle.bf16(np.float32([amax]))[0]
        s = np.float32(amax) / np.float32(127)
        k = np.arange(0, 127, dtype=np.float32) + np.float32(0.5)
        base = (k * s).astype(np.float32)
        cand = []
        for d in range(-6, 7):
            cand.append((base.view(np.int32) + d).view(np.float32))
        v = np.concatenate(cand + [-c for c in cand])
        v = v[np.abs(v) <= amax]
        if carrier == "bf16":
            v = np.unique(oracle.bf16(v))
        row = np.zeros(4096, np.float32)
        take = min(v.size, 4000)
        row[:take] = rng.permutation(v)[:take]
        row[4095] = amax
        rows.append(row)
    x = np.stack(rows)
    q, s = run_quantize(ops, x, carrier)
    eq, es = oracle.quantize(x)
    assert np.array_equal(bits(s), bits(es))
    assert np.array_equal(q, eq), int((q != eq).sum())


def test_quantizer_launch_with_prefetch_hints_changes_nothing(ops):
    """Few-row quantizer launches carry pending L2 prefetch hints as extra CTAs; codes and scales are unchanged, and a
    many-row launch leaves the hints for a later one."""
    import torch

    rng = np.random.default_rng(8)
    weights = torch.zeros(5 << 20, dtype=torch.int8, device="cuda")
    for M, K in [(1, 4096), (3, 12288)]:
        x = synth_activations(rng, M, K)
        gamma = synth_gamma(rng, K)
        xd, gd = to_dev(x, "bf16"), to_dev(gamma, "bf16")
        results = []
        for hinted in (False, True):
            out = []
            for kind in ("plain", "norm", "with_max"):
                if hinted:
                    ops.prefetch_hint(weights, 128, (4 << 20) + 5)
                q = torch.zeros((M, K), dtype=torch.int8, device="cuda")
                s = torch.zeros((M,), dtype=torch.float32, device="cuda")
                if kind == "plain":
                    ops.quantize(xd, q, s)
                elif kind == "norm":
                    ops.norm_quantize(xd, gd, None, q, s, None)
                else:
                    mx = to_dev(np.abs(x).max(1).astype(np.float32).view(np.uint32))
                    ops.quantize_with_max(xd, mx, q, s)
                out.append((to_host(q), to_host(s)))
            results.append(out)
        for (q0, s0), (q1, s1) in zip(*results):
            assert np.array_equal(q0, q1) and np.array_equal(bits(s0), bits(s1))
    eq, es = oracle.quantize(x)
    assert np.array_equal(results[0][0][0], eq)
    assert ops.device_status() == (0, 0)
