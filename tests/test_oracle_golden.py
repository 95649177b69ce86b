"""Pins the CPU oracle (oracle/w8a8_oracle.c) to the reference's own golden vectors:
the outputs of tools/operator_fixtures.py (PyTorch CPU, seed 824) committed under
tests/golden/operator_fixtures/, plus the closed-form known-answer tests of
src/conformance.rs (rounding boundaries :841-871)."""
import numpy as np

from oracle import oracle


def gate(actual, expected):
    """The reference's numeric gate (src/conformance.rs:658-674, docs/qwen3-8b-w8a8/coverage.md:28)."""
    a = actual.astype(np.float64).ravel()
    e = expected.astype(np.float64).ravel()
    assert np.all(np.abs(a - e) <= 2e-4 + 0.01 * np.abs(e))
    denom = np.linalg.norm(e)
    if denom > 0:
        assert np.linalg.norm(a - e) / denom <= 0.005


def test_quantize_cases_bit_exact(fixtures):
    cases = fixtures.cases("quantize")
    assert [c["width"] for c in cases] == [128, 4096, 12288]
    for c in cases:
        x = fixtures.tensor(c, "x")
        q, s = oracle.quantize(x)
        assert np.array_equal(q, fixtures.tensor(c, "q")), c["name"]
        assert np.array_equal(s.view(np.uint32), fixtures.tensor(c, "scale").reshape(-1).view(np.uint32)), c["name"]
        # zero row: scale floor 1e-8/127, all-zero codes (tools/operator_fixtures.py:39,43)
        assert s[0] == np.float32(1e-8) / np.float32(127) and not q[0].any()
        # tie values +-0.5,+-1.5,+-2.5 and +-127 in row 1 (tools/operator_fixtures.py:42)
        assert q[1, 0] == 127 and q[1, 1] == -127


def test_quantize_with_max_equals_quantize(fixtures):
    for c in fixtures.cases("quantize"):
        x = fixtures.tensor(c, "x")
        m = np.maximum(np.abs(x).max(-1), np.float32(1e-8)).astype(np.float32)
        q, s = oracle.quantize_with_max(x, m.view(np.uint32))
        assert np.array_equal(q, fixtures.tensor(c, "q"))
        assert np.array_equal(s, fixtures.tensor(c, "scale").reshape(-1))


def test_linear_cases_bit_exact(fixtures):
    cases = fixtures.cases("linear")
    assert [(c["width"], fixtures.tensor(c, "q").shape[0]) for c in cases] == [
        (4096, 1), (4096, 17), (12288, 3), (4096, 65), (12288, 129)]
    for c in cases:
        q, w = fixtures.tensor(c, "q"), fixtures.tensor(c, "w")
        asc, ws = fixtures.tensor(c, "asc"), fixtures.tensor(c, "ws")
        y = oracle.linear(q, asc, w, ws)
        expected = fixtures.tensor(c, "out")
        assert np.array_equal(y.view(np.uint32), expected.view(np.uint32)), c["name"]
        # worst-case accumulator the fixture plants (tools/operator_fixtures.py:50-51)
        acc = oracle.linear_acc(q, w)
        assert acc[0, 0] == c["width"] * 127 * 127 and acc[0, 1] == -c["width"] * 127 * 127
        assert np.array_equal(acc, q.astype(np.int64) @ w.astype(np.int64).T)
        # threads do not change anything
        assert np.array_equal(acc, oracle.linear_acc(q, w, threads=1))


def test_linear_residual_order(fixtures):
    # src/conformance.rs:220-225: residual operand ((i mod 17) - 8) * 0.0625; combined = bf16(residual + bf16(y))
    c = fixtures.cases("linear")[1]
    q, w = fixtures.tensor(c, "q"), fixtures.tensor(c, "w")
    asc, ws = fixtures.tensor(c, "asc"), fixtures.tensor(c, "ws")
    M, N = q.shape[0], w.shape[0]
    res = (((np.arange(M * N) % 17) - 8) * 0.0625).astype(np.float32).reshape(M, N)
    y, comb = oracle.linear(q, asc, w, ws, residual_in=res)
    assert np.array_equal(y, fixtures.tensor(c, "out"))
    assert np.array_equal(comb, oracle.bf16(res + y))
    assert np.array_equal(comb, oracle.residual(res, y))


def test_residual_case_bit_exact(fixtures):
    (c,) = fixtures.cases("residual")
    out = oracle.residual(fixtures.tensor(c, "a"), fixtures.tensor(c, "b"))
    assert np.array_equal(out.view(np.uint32), fixtures.tensor(c, "out").view(np.uint32))


def test_norm_cases_numeric_gate(fixtures):
    for c in fixtures.cases("norm"):
        y = oracle.rmsnorm(fixtures.tensor(c, "x"), fixtures.tensor(c, "gain"))
        gate(y, fixtures.tensor(c, "out"))
        assert np.array_equal(y, oracle.bf16(y))  # bf16-representable


def test_swiglu_case_numeric_gate(fixtures):
    (c,) = fixtures.cases("swiglu")
    act, mx = oracle.swiglu(fixtures.tensor(c, "gate"), fixtures.tensor(c, "up"))
    gate(act, fixtures.tensor(c, "out"))
    finite = np.abs(act[np.isfinite(act)])
    assert mx == max(np.float32(1e-8), finite.max()).view(np.uint32)


def rounding_inputs() -> np.ndarray:
    """The 1 328 443 inputs of src/conformance.rs:843-857."""
    parts = [(np.arange(65536, dtype=np.uint32) << np.uint32(16)).view(np.float32),
             (np.arange(-131072, 131073, dtype=np.int64) / 1024.0).astype(np.float32)]
    ties = []
    for i in range(-127, 127):
        b = np.float32(i + 0.5).view(np.uint32)
        ties += [b - np.uint32(1), b, b + np.uint32(1)]
    parts.append(np.array(ties, dtype=np.uint32).view(np.float32))
    parts.append((np.arange(1_000_000, dtype=np.uint64) * np.uint64(2654435761) & np.uint64(0xFFFFFFFF))
                 .astype(np.uint32).view(np.float32))
    return np.concatenate(parts)


def rounding_expected(x: np.ndarray) -> np.ndarray:
    """f64.clamp(+-127).round_ties_even() as i8 (src/conformance.rs:858-861); NaN casts to 0."""
    d = x.astype(np.float64)
    with np.errstate(invalid="ignore"):
        r = np.rint(np.clip(d, -127.0, 127.0))
    r[np.isnan(r)] = 0
    return r.astype(np.int8)


def test_integer_rounding_boundaries():
    x = rounding_inputs()
    assert x.size == 1_328_443
    assert np.array_equal(oracle.round_i8(x), rounding_expected(x))


def test_bf16_matches_numpy_vectorised_and_scalar():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(10000).astype(np.float32) * 100
    v = oracle.bf16(x)
    s = np.array([oracle.lib().oracle_bf16(float(t)) for t in x[:500]], np.float32)
    assert np.array_equal(v[:500], s)
    # ties to even on the 16-bit boundary
    assert oracle.bf16(np.array([np.uint32(0x3F808000)], np.uint32).view(np.float32)).view(np.uint32)[0] == 0x3F800000
    assert oracle.bf16(np.array([np.uint32(0x3F818000)], np.uint32).view(np.float32)).view(np.uint32)[0] == 0x3F820000


def test_weight_quantize_is_row_quantize():
    # tools/prepare.py:79-81 is the same formula as the activation quantizer, per output channel
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((33, 256)) * 0.02).astype(np.float32)
    q, s = oracle.weight_quantize(w)
    assert np.array_equal(s, np.maximum(np.abs(w).max(1), np.float32(1e-8)) / np.float32(127))
    assert np.array_equal(q, np.clip(np.rint(w / s[:, None]), -127, 127).astype(np.int8))
    assert np.abs(q).max() == 127


# ---- the operators around the linear layers ---------------------------------------------------------------

def reference_tolerance(expected: np.ndarray) -> np.ndarray:
    """Per-element bound of the reference's own fixture test for non-exact operators (src/conformance.rs:661)."""
    return 2e-4 + 0.01 * np.abs(expected)


def test_rope_matches_reference_fixture_exactly(fixtures):
    # `rope` is one of the operators the reference compares exactly (src/conformance.rs:658)
    (case,) = fixtures.cases("rope")
    x = fixtures.tensor(case, "x")
    rows = fixtures.tensor(case, "table_rows")
    table = np.zeros((case["position"] + x.shape[0], 128), np.float32)
    table[case["position"]:] = rows
    assert np.array_equal(oracle.rope(x, table, case["position"]), fixtures.tensor(case, "out"))


def test_embedding_matches_reference_fixture_exactly(fixtures):
    (case,) = fixtures.cases("embedding")
    got = oracle.embedding(fixtures.tensor(case, "ids"), fixtures.tensor(case, "w"))
    assert np.array_equal(got, fixtures.tensor(case, "out"))


def test_attention_within_reference_tolerance(fixtures):
    cases = fixtures.cases("attention")
    assert [c["position"] for c in cases] == [0, 129]
    for case in cases:
        expected = fixtures.tensor(case, "out")
        got = oracle.attention(fixtures.tensor(case, "q"), fixtures.tensor(case, "k"), fixtures.tensor(case, "v"), case["position"])
        assert np.all(np.abs(got - expected) <= reference_tolerance(expected))
        rel = np.sqrt(((got.astype(np.float64) - expected) ** 2).sum() / (expected.astype(np.float64) ** 2).sum())
        assert rel <= 0.005  # src/conformance.rs:669-673


def test_head_norm_is_the_fixture_pinned_norm_at_width_128(fixtures):
    """The fused head norm + rope is defined by the reference as `norm` (width 128) followed by `rope`
    (src/conformance.rs:375-401); the width-128 norm is pinned by the reference's norm fixture, and the numpy
    restatement of the head norm equals the C restatement of `norm` bit for bit."""
    (case,) = [c for c in fixtures.cases("norm") if c["width"] == 128]
    x, gain = fixtures.tensor(case, "x"), fixtures.tensor(case, "gain")
    assert np.array_equal(oracle.head_norm(x, gain), oracle.rmsnorm(x.reshape(-1, 128), gain).reshape(x.shape))
    rng = np.random.default_rng(5)
    y = oracle.bf16((rng.standard_normal((300, 8, 128)) * rng.uniform(0.01, 30, (300, 8, 1))).astype(np.float32))
    g = (1 + 0.2 * rng.standard_normal(128)).astype(np.float32)
    assert np.array_equal(oracle.head_norm(y, g), oracle.rmsnorm(y.reshape(-1, 128), g).reshape(y.shape))
    moved = oracle.head_norm(y, g, inv_ulps=2)
    assert 0 < (moved != oracle.head_norm(y, g)).mean() < 0.02


def test_head_restatement_against_the_reference_fixture(fixtures):
    """`head` (src/kernels.rs:2233-2257) restated with the kernel's summation order: inside the reference's gate for the
    operator against its Torch-generated fixture (src/conformance.rs:611-674; in fact equal on all 33 logits)."""
    from tests.util import gate

    (case,) = fixtures.cases("head")
    x = fixtures.tensor(case, "x")
    w_bits = np.frombuffer((fixtures.root / case["tensors"]["w"]["file"]).read_bytes(), np.uint16).reshape(case["tensors"]["w"]["shape"])
    expected = fixtures.tensor(case, "out").reshape(-1)
    got = oracle.head(x[-1], w_bits)
    gate(got, expected)
    assert np.array_equal(got, oracle.bf16(got))  # logits are bf16 values
