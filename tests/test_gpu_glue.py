"""GPU parity of the operators around the linear layers (include/qwen3_glue.h) through the C ABI: against the
reference's fixtures and against the CPU restatement on seeded inputs."""
import numpy as np
import pytest

from oracle import oracle
from tests.util import to_dev, to_host

pytestmark = pytest.mark.gpu

Q_HEADS, KV_HEADS = 32, 8


@pytest.fixture(scope="module")
def ops():
    from inferrous_b200 import ops as o

    o.init()
    return o


def control(token: int, position: int):
    return to_dev(np.array([token, position], np.uint32))


def table_for(positions: int, seed: int = 3) -> np.ndarray:
    rng = np.random.default_rng(seed)
    angles = rng.uniform(0, 6.28, (positions, 64)).astype(np.float32)
    return np.concatenate([np.cos(angles), np.sin(angles)], 1).astype(np.float32)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_embedding_fixture(ops, fixtures, dtype):
    import torch

    (case,) = fixtures.cases("embedding")
    ids = to_dev(fixtures.tensor(case, "ids"))
    table = to_dev(fixtures.tensor(case, "w").view(np.int16)).view(torch.bfloat16)
    expected = fixtures.tensor(case, "out")
    out = torch.full(expected.shape, float("nan"), dtype=torch.bfloat16 if dtype == "bf16" else torch.float32, device="cuda")
    ops.embedding(ids, table, out)
    assert np.array_equal(to_host(out), expected)
    assert ops.device_status() == (0, 0)


def test_embedding_rejects_a_bad_id_without_touching_memory(ops):
    import torch

    table = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    out = torch.full((2, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.embedding(to_dev(np.array([1, 9], np.uint32)), table, out)
    status, detail = ops.device_status()
    assert status != 0 and detail >> 24 == 6 and (detail & 0xFFFFFF) == 9
    assert float(out[1].float().min()) == 7.0 and float(out[0].float().max()) == 0.0
    assert ops.device_status() == (0, 0)  # reading clears it


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("rows,position", [(1, 0), (3, 4093), (129, 7)])
def test_prepare_qk_matches_norm_then_rope(ops, dtype, rows, position):
    """Queries and keys in place, keys and values in the cache; the cache holds exactly the in-place keys."""
    import torch

    rng = np.random.default_rng(rows + position)
    capacity = 4096
    width = (Q_HEADS + 2 * KV_HEADS) * 128
    x = oracle.bf16((rng.standard_normal((rows, width)) * 3).astype(np.float32))
    qg = ((np.arange(128) % 13 - 6) * 0.25).astype(np.float32)  # the gains of src/conformance.rs:377-381
    kg = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    table = np.zeros((capacity, 128), np.float32)
    table[position:position + rows] = table_for(rows)
    qkv = to_dev(x, dtype)
    kc = torch.zeros(capacity, KV_HEADS, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    ops.prepare_qk(qkv, Q_HEADS, KV_HEADS, to_dev(qg), to_dev(kg), to_dev(table), control(0, position), kc, vc)
    got = to_host(qkv)
    q_in = x[:, :Q_HEADS * 128].reshape(rows, Q_HEADS, 128)
    k_in = x[:, Q_HEADS * 128:(Q_HEADS + KV_HEADS) * 128].reshape(rows, KV_HEADS, 128)
    v_in = x[:, (Q_HEADS + KV_HEADS) * 128:].reshape(rows, KV_HEADS, 128)
    got_q = got[:, :Q_HEADS * 128].reshape(rows, Q_HEADS, 128)
    got_k = got[:, Q_HEADS * 128:(Q_HEADS + KV_HEADS) * 128].reshape(rows, KV_HEADS, 128)
    k_exp = got_k
    for heads_in, gains, heads_out in ((q_in, qg, got_q), (k_in, kg, got_k)):
        # Every head must equal the restatement exactly for ONE value of inv within the error of rsqrt.approx
        # (a few float32 steps from the correctly rounded 1/sqrt); most heads need no correction at all.
        candidates = {u: oracle.head_norm_rope(heads_in, gains, table, position, inv_ulps=u) for u in (0, -1, 1, -2, 2, -3, 3)}
        explained = np.zeros(heads_out.shape[:2], bool)
        for cand in candidates.values():
            explained |= (cand == heads_out).all(-1)
        assert explained.all(), np.argwhere(~explained)[:5]
        assert (candidates[0] == heads_out).all(-1).mean() > 0.5
    assert np.array_equal(got[:, (Q_HEADS + KV_HEADS) * 128:], x[:, (Q_HEADS + KV_HEADS) * 128:])  # values untouched
    kc_h, vc_h = to_host(kc), to_host(vc)
    assert np.array_equal(kc_h[position:position + rows], k_exp)
    assert np.array_equal(vc_h[position:position + rows], v_in)
    mask = np.ones(capacity, bool)
    mask[position:position + rows] = False
    assert not kc_h[mask].any() and not vc_h[mask].any()
    assert ops.device_status() == (0, 0)


def test_prepare_qk_skips_positions_beyond_the_cache(ops):
    import torch

    capacity = 8
    qkv = torch.ones(2, (4 + 2 * 2) * 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(capacity, 2, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    gains = torch.ones(128, device="cuda")
    table = torch.zeros(capacity, 128, device="cuda")
    ops.prepare_qk(qkv, 4, 2, gains, gains, table, control(0, 7), kc, vc)  # row 1 would land on position 8
    status, detail = ops.device_status()
    assert status != 0 and detail >> 24 == 6 and (detail & 0xFFFFFF) == 8
    assert float(vc[7].float().min()) == 1.0  # row 0 was appended


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_attention_fixtures(ops, fixtures, dtype):
    import torch

    for case in fixtures.cases("attention"):
        q = fixtures.tensor(case, "q")
        k = fixtures.tensor(case, "k")
        v = fixtures.tensor(case, "v")
        expected = fixtures.tensor(case, "out")
        rows, position = q.shape[0], case["position"]
        capacity = 256
        kc = torch.zeros(capacity, KV_HEADS, 128, dtype=torch.bfloat16, device="cuda")
        vc = torch.zeros_like(kc)
        kc[:k.shape[0]] = to_dev(k.view(np.int16)).view(torch.bfloat16)
        vc[:v.shape[0]] = to_dev(v.view(np.int16)).view(torch.bfloat16)
        out = torch.full((rows, Q_HEADS * 128), float("nan"), dtype=torch.bfloat16 if dtype == "bf16" else torch.float32,
                         device="cuda")
        ops.attention(to_dev(q.reshape(rows, -1), dtype), Q_HEADS, KV_HEADS, kc, vc, control(0, position), out)
        got = to_host(out).reshape(expected.shape)
        # the reference's own bound for this operator (src/conformance.rs:661, 669-673)
        assert np.all(np.abs(got - expected) <= 2e-4 + 0.01 * np.abs(expected))
        rel = np.sqrt(((got.astype(np.float64) - expected) ** 2).sum() / (expected.astype(np.float64) ** 2).sum())
        assert rel <= 0.005
        # against the CPU restatement of the reference kernel (sequential float32 sums, correctly rounded exp): the
        # GPU kernel reassociates the sums and uses ex2.approx, which moves a result by at most one bf16 step and
        # leaves nearly every element identical
        cpu = oracle.attention(q, k, v, position)
        assert np.all(np.abs(got - cpu) <= np.abs(cpu) * 2.0 ** -7 + 5e-6)
        assert (got != cpu).mean() < 0.05
    assert ops.device_status() == (0, 0)


def test_attention_strided_query_and_small_head_counts(ops):
    """q read out of a wider qkv buffer; 4 query heads on 2 key heads; 5 rows at position 3."""
    import torch

    rng = np.random.default_rng(11)
    rows, position, qh, kvh = 5, 3, 4, 2
    width = (qh + 2 * kvh) * 128
    x = oracle.bf16(rng.standard_normal((rows, width)).astype(np.float32))
    keys = position + rows
    k = oracle.bf16_bits(rng.standard_normal((keys, kvh, 128)).astype(np.float32))
    v = oracle.bf16_bits(rng.standard_normal((keys, kvh, 128)).astype(np.float32))
    kc = torch.zeros(16, kvh, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    kc[:keys] = to_dev(k.view(np.int16)).view(torch.bfloat16)
    vc[:keys] = to_dev(v.view(np.int16)).view(torch.bfloat16)
    out = torch.full((rows, qh * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.attention(to_dev(x, "bf16"), qh, kvh, kc, vc, control(0, position), out)
    cpu = oracle.attention(x[:, :qh * 128].reshape(rows, qh, 128), k, v, position)
    got = to_host(out).reshape(cpu.shape)
    assert np.all(np.abs(got - cpu) <= np.abs(cpu) * 2.0 ** -7 + 5e-6)
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("rows,position", [(1, 1500), (2, 700), (1, 63), (1, 64)])
def test_attention_split_over_several_ctas(ops, rows, position):
    """Few rows: the keys of each (row, head) are split over several CTAs and combined by the last one to arrive.
    Same bound as above against the sequential CPU restatement; a second launch (the arrival counters must be back
    at zero) gives the same bits."""
    import torch

    rng = np.random.default_rng(position)
    keys = position + rows
    q = oracle.bf16(rng.standard_normal((rows, Q_HEADS, 128)).astype(np.float32))
    k = oracle.bf16_bits((rng.standard_normal((keys, KV_HEADS, 128)) * 0.7).astype(np.float32))
    v = oracle.bf16_bits(rng.standard_normal((keys, KV_HEADS, 128)).astype(np.float32))
    kc = torch.zeros(2048, KV_HEADS, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    kc[:keys] = to_dev(k.view(np.int16)).view(torch.bfloat16)
    vc[:keys] = to_dev(v.view(np.int16)).view(torch.bfloat16)
    qd = to_dev(q.reshape(rows, -1), "bf16")
    outs = []
    for _ in range(2):
        out = torch.full((rows, Q_HEADS * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        mx = to_dev(np.full(rows, np.float32(1e-8).view(np.uint32), np.uint32))
        ops.attention(qd, Q_HEADS, KV_HEADS, kc, vc, control(0, position), out, mx)
        outs.append(to_host(out))
        # the published maximum is the row's max |out|
        assert np.array_equal(to_host(mx).view(np.uint32), np.abs(outs[-1]).max(1).astype(np.float32).view(np.uint32))
    assert np.array_equal(outs[0], outs[1])
    cpu = oracle.attention(q, k, v, position).reshape(rows, -1)
    assert np.all(np.abs(outs[0] - cpu) <= np.abs(cpu) * 2.0 ** -7 + 5e-6)
    assert (outs[0] != cpu).mean() < 0.05
    assert ops.device_status() == (0, 0)


def test_attention_with_prefetch_hints_changes_nothing(ops):
    """A launch that carries L2 prefetch CTAs for some weight ranges computes the same bits; the hints are consumed."""
    import torch

    rng = np.random.default_rng(4)
    position, keys = 300, 301
    q = to_dev(oracle.bf16(rng.standard_normal((1, Q_HEADS * 128)).astype(np.float32)), "bf16")
    kc = to_dev(oracle.bf16(rng.standard_normal((512, KV_HEADS, 128)).astype(np.float32)), "bf16")
    vc = to_dev(oracle.bf16(rng.standard_normal((512, KV_HEADS, 128)).astype(np.float32)), "bf16")
    weights = torch.zeros(3 << 20, dtype=torch.int8, device="cuda")
    outs = []
    for hinted in (False, True, False):
        if hinted:
            ops.prefetch_hint(weights, 0, 1 << 20)
            ops.prefetch_hint(weights, (2 << 20) + 128, (1 << 20) - 128 - 77)  # an end that is not a multiple of a line
        out = torch.full((1, Q_HEADS * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.attention(q, Q_HEADS, KV_HEADS, kc, vc, control(0, position), out)
        outs.append(to_host(out))
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("rows,position,qh,kvh", [(70, 50, 32, 8), (33, 0, 4, 2), (200, 3, 8, 2)])
def test_attention_on_tensor_cores(ops, dtype, rows, position, qh, kvh):
    """Launches of 32 rows or more take the tensor-core kernel: the same bound against the sequential CPU restatement as
    the CUDA-core kernels, the same published maxima rule, and agreement with the CUDA-core kernel on the same inputs
    to within one bf16 step."""
    import torch

    rng = np.random.default_rng(rows * 7 + position)
    keys = position + rows
    q = oracle.bf16(rng.standard_normal((rows, qh, 128)).astype(np.float32))
    k = oracle.bf16_bits((rng.standard_normal((keys, kvh, 128)) * 0.8).astype(np.float32))
    v = oracle.bf16_bits(rng.standard_normal((keys, kvh, 128)).astype(np.float32))
    capacity = 256
    kc = torch.full((capacity, kvh, 128), float("nan"), dtype=torch.bfloat16, device="cuda")  # unwritten slots must not leak
    vc = torch.full((capacity, kvh, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    kc[:keys] = to_dev(k.view(np.int16)).view(torch.bfloat16)
    vc[:keys] = to_dev(v.view(np.int16)).view(torch.bfloat16)
    qd = to_dev(q.reshape(rows, -1), dtype)
    td = torch.bfloat16 if dtype == "bf16" else torch.float32
    results = {}
    for tensor_cores in (True, False):
        ops.attention_use_tensor_cores(tensor_cores)
        try:
            out = torch.full((rows, qh * 128), float("nan"), dtype=td, device="cuda")
            mx = to_dev(np.full(rows, np.float32(1e-8).view(np.uint32), np.uint32))
            ops.attention(qd, qh, kvh, kc, vc, control(0, position), out, mx)
            got = to_host(out)
            assert np.array_equal(to_host(mx).view(np.uint32), np.abs(got).max(1).astype(np.float32).view(np.uint32))
            results[tensor_cores] = got
        finally:
            ops.attention_use_tensor_cores(True)
    cpu = oracle.attention(q, k, v, position).reshape(rows, -1)
    for got in results.values():
        assert np.all(np.abs(got - cpu) <= np.abs(cpu) * 2.0 ** -7 + 5e-6)
        assert (got != cpu).mean() < 0.05
    assert np.all(np.abs(results[True] - results[False]) <= np.abs(results[False]) * 2.0 ** -7 + 5e-6)
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("rows,position", [(1, 0), (1, 40), (1, 700), (3, 130)])
def test_attention_with_folded_quantizer(ops, dtype, rows, position):
    """Few rows: the attention launch also writes the int8 codes and the scale of its output row; they must be exactly
    what w8a8_quantize makes of that output, the output itself must be unchanged, and a second launch must agree."""
    import torch

    rng = np.random.default_rng(position + rows)
    keys = position + rows
    qd = to_dev(oracle.bf16(rng.standard_normal((rows, Q_HEADS * 128)).astype(np.float32)), dtype)
    kc = to_dev(oracle.bf16(rng.standard_normal((1024, KV_HEADS, 128)).astype(np.float32)), "bf16")
    vc = to_dev(oracle.bf16((rng.standard_normal((1024, KV_HEADS, 128)) * 3).astype(np.float32)), "bf16")
    td = torch.bfloat16 if dtype == "bf16" else torch.float32
    plain = torch.full((rows, Q_HEADS * 128), float("nan"), dtype=td, device="cuda")
    ops.attention(qd, Q_HEADS, KV_HEADS, kc, vc, control(0, position), plain)
    q_ref = torch.zeros((rows, Q_HEADS * 128), dtype=torch.int8, device="cuda")
    s_ref = torch.zeros(rows, dtype=torch.float32, device="cuda")
    ops.quantize(plain, q_ref, s_ref)
    for _ in range(2):
        out = torch.full_like(plain, float("nan"))
        codes = torch.full_like(q_ref, 99)
        scale = torch.zeros_like(s_ref)
        ops.attention_quantize(qd, Q_HEADS, KV_HEADS, kc, vc, control(0, position), out, codes, scale)
        assert torch.equal(out.view(torch.int16 if dtype == "bf16" else torch.int32), plain.view(torch.int16 if dtype == "bf16" else torch.int32))
        assert torch.equal(codes, q_ref)
        assert np.array_equal(to_host(scale).view(np.uint32), to_host(s_ref).view(np.uint32))
    eq, es = oracle.quantize(to_host(plain))
    assert np.array_equal(to_host(q_ref), eq) and np.array_equal(to_host(s_ref).view(np.uint32), es.view(np.uint32))
    assert ops.device_status() == (0, 0)


def test_attention_with_folded_quantizer_refuses_many_rows(ops):
    import torch

    from inferrous_b200 import capi

    rows = 8  # 8 rows x 32 heads is past the SM count: that launch takes another kernel
    qd = torch.zeros(rows, Q_HEADS * 128, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(64, KV_HEADS, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(qd)
    with pytest.raises(capi.W8A8Error) as e:
        ops.attention_quantize(qd, Q_HEADS, KV_HEADS, kc, kc, control(0, 0), out, torch.zeros(rows, Q_HEADS * 128, dtype=torch.int8, device="cuda"),
                               torch.zeros(rows, device="cuda"))
    assert e.value.status == 3


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_head_bf16_fixture_and_reference_order(ops, fixtures, dtype):
    """The reference's `head` fixture (x [3, 4096], w [33, 4096] bf16): the last row's logits inside the reference's gate
    for this operator (its expected values come from a Torch matmul, src/conformance.rs:611-674), and bit-identical to
    the CPU restatement of the kernel's own summation order (src/kernels.rs:2233-2257); the fused selection agrees."""
    import torch

    from tests.util import gate

    (case,) = fixtures.cases("head")
    x = fixtures.tensor(case, "x")
    w_bits = np.frombuffer((fixtures.root / case["tensors"]["w"]["file"]).read_bytes(), np.uint16).reshape(case["tensors"]["w"]["shape"])
    expected = fixtures.tensor(case, "out").reshape(-1)
    w = to_dev(w_bits.view(np.int16).copy()).view(torch.bfloat16)
    td = torch.bfloat16 if dtype == "bf16" else torch.float32
    logits = torch.full((w.shape[0],), float("nan"), dtype=td, device="cuda")
    token = torch.zeros(1, dtype=torch.int32, device="cuda")
    value = torch.zeros(1, dtype=torch.float32, device="cuda")
    ops.head_bf16(to_dev(x[-1:], dtype), w, logits, token, value)
    got = to_host(logits)
    gate(got, expected)
    cpu = oracle.head(x[-1], w_bits)
    assert np.array_equal(got.view(np.uint32), cpu.view(np.uint32))
    assert int(token[0]) == int(np.argmax(cpu)) and float(value[0]) == float(cpu.max())
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("vocab,hidden", [(1000, 4096), (151936, 4096), (17, 256), (640, 1024), (50, 992), (33, 288)])
def test_head_bf16_shapes_ties_and_bad_rows(ops, vocab, hidden):
    """Ragged vocabulary sizes (a last CTA with fewer than 16 rows), the full Qwen3 vocabulary, other widths: logits bit-identical
    to the CPU restatement; equal maxima go to the lowest index; an infinite logit gives 0xffffffff."""
    import torch

    rng = np.random.default_rng(vocab)
    x = oracle.bf16(rng.standard_normal(hidden).astype(np.float32))
    w = oracle.bf16((rng.standard_normal((vocab, hidden)) * 0.05).astype(np.float32))
    w[vocab // 2] = w[vocab // 3]  # two identical rows: identical logits
    w_bits = oracle.bf16_bits(w)
    wd = to_dev(w_bits.view(np.int16)).view(torch.bfloat16)
    logits = torch.full((vocab,), float("nan"), dtype=torch.bfloat16, device="cuda")
    token = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.head_bf16(to_dev(x.reshape(1, -1), "bf16"), wd, logits, token)
    rows = slice(None) if vocab <= 2000 else rng.choice(vocab, 2000, replace=False)
    cpu = oracle.head(x, w_bits[rows])
    got = to_host(logits)
    assert np.array_equal(got[rows].view(np.uint32), cpu.view(np.uint32))
    assert int(token[0]) == int(np.flatnonzero(got == got.max())[0])
    # make the tied rows the maximum: the lower index wins
    big = x.copy()
    w2 = w.copy()
    w2[vocab // 2] = w2[vocab // 3] = oracle.bf16(np.sign(x) * 0.5)
    wd2 = to_dev(oracle.bf16_bits(w2).view(np.int16)).view(torch.bfloat16)
    only_token = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.head_bf16(to_dev(big.reshape(1, -1), "bf16"), wd2, None, only_token)
    assert int(only_token[0]) == vocab // 3
    # a logit that overflows to infinity marks the row of activations as bad (a NaN sum, by contrast, becomes -0.0 in
    # the reference's bf16 rounding, which has no NaN case: src/kernels.rs:12-15)
    x[0] = float(oracle.bf16(np.array([3e38], np.float32))[0])
    w3 = w.copy()
    w3[5, 0] = x[0]
    wd3 = to_dev(oracle.bf16_bits(w3).view(np.int16)).view(torch.bfloat16)
    ops.head_bf16(to_dev(x.reshape(1, -1), "f32"), wd3, None, only_token)
    assert int(only_token[0]) & 0xFFFFFFFF == 0xFFFFFFFF
    assert ops.device_status() == (0, 0)
