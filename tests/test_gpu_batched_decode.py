"""Batched ("ragged") decode through the C ABI: every row of a step is the newest token of its own sequence, with its own
position and its own KV cache.  Kernel level: the batched operators against the single-sequence ones and the CPU
restatement.  Model level: sequences decoded side by side give the bits they give when decoded alone."""
import numpy as np
import pytest

from oracle import oracle
from tests.util import to_dev, to_host

pytestmark = pytest.mark.gpu

F32_1E8 = int(np.float32(1e-8).view(np.uint32))


@pytest.fixture(scope="module")
def ops():
    from inferrous_b200 import ops as o

    o.init()
    return o


def random_caches(rng, sequences, capacity, kv_heads):
    import torch

    k = oracle.bf16_bits((rng.standard_normal((sequences, capacity, kv_heads, 128)) * 0.7).astype(np.float32))
    v = oracle.bf16_bits(rng.standard_normal((sequences, capacity, kv_heads, 128)).astype(np.float32))
    kc = to_dev(k.view(np.int16)).view(torch.bfloat16)
    vc = to_dev(v.view(np.int16)).view(torch.bfloat16)
    return k, v, kc, vc


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("qh,kvh,positions", [
    (32, 8, [0, 31, 32, 127, 128, 511, 512, 700, 1024, 1025, 2047]),   # one step, one warp, one unit, exact multiples, a unit of one key
    (8, 2, [5, 4095, 300]),                                  # the longest context: 8 units of 512 keys
    (16, 2, [77, 1500]),                                     # eight query heads per key/value head
    (4, 4, [90, 91]),                                        # one query head per key/value head
    (6, 3, [513, 2]),                                        # two query heads per key/value head
])
def test_attention_batched_matches_the_cpu_restatement(ops, dtype, qh, kvh, positions):
    """Row r attends to keys 0 .. positions[r] of sequence r's cache: same bound against the sequential CPU restatement
    as the single-sequence kernels, published row maxima, counters back at zero (a second launch gives the same bits),
    and every row equal to the same row launched alone (the split of the keys depends on the context length only)."""
    import torch

    rows = len(positions)
    capacity = 4096 if max(positions) >= 2048 else 2048
    rng = np.random.default_rng(rows * 1000 + qh)
    k, v, kc, vc = random_caches(rng, rows, capacity, kvh)
    q = oracle.bf16(rng.standard_normal((rows, qh, 128)).astype(np.float32))
    qd = to_dev(q.reshape(rows, -1), dtype)
    pos = to_dev(np.array(positions, np.uint32))
    ws = ops.attention_batched_workspace(rows, qh, kvh)
    td = torch.bfloat16 if dtype == "bf16" else torch.float32
    outs = []
    for _ in range(2):
        out = torch.full((rows, qh * 128), float("nan"), dtype=td, device="cuda")
        mx = to_dev(np.full(rows, F32_1E8, np.uint32))
        ops.attention_batched(qd, qh, kvh, kc, vc, pos, out, ws, mx)
        outs.append(to_host(out))
        assert np.array_equal(to_host(mx).view(np.uint32), np.abs(outs[-1]).max(1).astype(np.float32).view(np.uint32))
    assert np.array_equal(outs[0], outs[1])
    for r, p in enumerate(positions):
        cpu = oracle.attention(q[r:r + 1], k[r], v[r], p).reshape(-1)
        assert np.all(np.abs(outs[0][r] - cpu) <= np.abs(cpu) * 2.0 ** -7 + 5e-6), (r, p)
        alone = torch.full((1, qh * 128), float("nan"), dtype=td, device="cuda")
        ops.attention_batched(qd[r:r + 1], qh, kvh, kc[r:r + 1], vc[r:r + 1], pos[r:r + 1], alone,
                              ops.attention_batched_workspace(1, qh, kvh))
        assert np.array_equal(to_host(alone)[0], outs[0][r]), (r, p)
    assert ops.device_status() == (0, 0)


def test_attention_batched_workspace_counters_only(ops):
    """The workspace's leading words are ticket and arrival counters that every launch leaves at zero; what follows are
    partial results that the next launch overwrites before it reads them."""
    import torch

    rng = np.random.default_rng(5)
    rows, qh, kvh = 3, 8, 2
    _, _, kc, vc = random_caches(rng, rows, 2048, kvh)
    qd = to_dev(oracle.bf16(rng.standard_normal((rows, qh * 128)).astype(np.float32)), "bf16")
    pos = to_dev(np.array([1400, 70, 3], np.uint32))  # the first row has three units, whose partial results meet in the workspace
    ws = ops.attention_batched_workspace(rows, qh, kvh)
    out = torch.empty((rows, qh * 128), dtype=torch.bfloat16, device="cuda")
    ops.attention_batched(qd, qh, kvh, kc, vc, pos, out, ws)
    first = to_host(out).copy()
    counters = 256 // 4 + (rows * qh * 4 + 255) // 256 * 256 // 4  # one 256-byte block of tickets, then the arrival counters
    assert not ws[:counters].any() and ws[counters:].any()
    ws[counters:].fill_(0x7FC00000)  # NaN in every partial result: a launch must not read what it has not written
    ops.attention_batched(qd, qh, kvh, kc, vc, pos, out, ws)
    assert np.array_equal(to_host(out), first)


def test_attention_batched_skips_a_position_beyond_the_cache(ops):
    import torch

    rng = np.random.default_rng(6)
    _, _, kc, vc = random_caches(rng, 2, 256, 2)
    qd = to_dev(oracle.bf16(rng.standard_normal((2, 4 * 128)).astype(np.float32)), "bf16")
    out = torch.full((2, 4 * 128), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.attention_batched(qd, 4, 2, kc, vc, to_dev(np.array([10, 256], np.uint32)), out, ops.attention_batched_workspace(2, 4, 2))
    status, detail = ops.device_status()
    assert status != 0 and detail >> 24 == 6 and (detail & 0xFFFFFF) == 257
    got = to_host(out)
    assert np.all(got[1] == 7.0) and not np.any(got[0] == 7.0)
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_prepare_qk_batched_equals_one_call_per_sequence(ops, dtype):
    """Row r rotated with the table row of positions[r] and appended to sequence r's caches: bit for bit what
    qwen3_prepare_qk does for that row alone at that position."""
    import torch

    rng = np.random.default_rng(8)
    qh, kvh, capacity = 8, 2, 128
    positions = [0, 127, 5, 64, 31]
    rows = len(positions)
    width = (qh + 2 * kvh) * 128
    x = oracle.bf16(rng.standard_normal((rows, width)).astype(np.float32))
    qg = to_dev((1.0 + 0.1 * rng.standard_normal(128)).astype(np.float32))
    kg = to_dev((1.0 + 0.1 * rng.standard_normal(128)).astype(np.float32))
    angles = rng.uniform(0, 6.28, (capacity, 64)).astype(np.float32)
    table = to_dev(np.concatenate([np.cos(angles), np.sin(angles)], 1).astype(np.float32))
    kc = torch.zeros(rows, capacity, kvh, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    batched = to_dev(x, dtype)
    ops.prepare_qk_batched(batched, qh, kvh, qg, kg, table, to_dev(np.array(positions, np.uint32)), kc, vc)
    for r, p in enumerate(positions):
        one = to_dev(x[r:r + 1], dtype)
        k1 = torch.zeros(capacity, kvh, 128, dtype=torch.bfloat16, device="cuda")
        v1 = torch.zeros_like(k1)
        ops.prepare_qk(one, qh, kvh, qg, kg, table, to_dev(np.array([0, p], np.uint32)), k1, v1)
        assert np.array_equal(to_host(one)[0], to_host(batched)[r])
        assert np.array_equal(to_host(k1), to_host(kc[r])) and np.array_equal(to_host(v1), to_host(vc[r]))
        assert float(kc[r, p].float().abs().max()) > 0
    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("n,ld", [(151936, 151936), (1000, 1003), (7, 8), (4096, 4096)])
def test_select_token_rule(ops, dtype, n, ld):
    """Largest value, lowest index among equals (+0.0 and -0.0 are equal), 0xffffffff for a row with a non-finite logit
    (select_token, src/kernels.rs:2191-2231; host check model::argmax, src/model.rs:206-218)."""
    import torch

    rng = np.random.default_rng(n)
    rows = 6
    x = oracle.bf16(rng.standard_normal((rows, ld)).astype(np.float32))
    x[1, [n // 2, n - 1]] = x[1, :n].max() + 1.0          # a tie: the lower index wins
    x[2, :n] = -0.0
    x[2, n // 3] = 0.0                                     # all equal: index 0
    x[3, n - 1] = np.inf
    x[4, 0] = np.nan
    x[5, :n] = -np.abs(x[5, :n]) - 1.0                     # all negative
    if ld > n:
        x[:, n:] = 1e30                                    # padding beyond n must not be read as a logit
    finite = np.isfinite(x)
    x[finite] = oracle.bf16(x[finite])                     # what the bf16 carrier stores
    token = torch.full((rows,), 77, dtype=torch.int32, device="cuda")
    value = torch.full((rows,), 77.0, dtype=torch.float32, device="cuda")
    ops.select_token(to_dev(x, dtype)[:, :n], token, value)
    got = to_host(token).view(np.uint32)
    vals = to_host(value)
    for r in range(rows):
        row = x[r, :n]
        if not np.isfinite(row).all():
            assert got[r] == 0xFFFFFFFF and np.isnan(vals[r])
        else:
            assert got[r] == int(np.argmax(row)) and vals[r] == row.max()
    assert got[1] == n // 2 and got[2] == 0


def test_merge_candidates(ops):
    import torch

    parts, rows, width = 4, 5, 1000
    tokens = np.array([[1, 2, 3, 4, 5], [10, 20, 30, 40, 50], [7, 7, 7, 7, 7], [9, 9, 9, 0xFFFFFFFF, 9]], np.uint32)
    values = np.array([[1.0, 5.0, -1.0, 0.0, 2.0], [2.0, 5.0, -3.0, 0.0, 2.0], [0.5, 4.0, -0.5, 0.0, np.inf], [2.0, 5.0, -2.0, 0.0, 1.0]],
                      np.float32)
    cand = np.stack([tokens, values.view(np.uint32)], 1)  # [parts, 2, rows]
    assert cand.shape == (parts, 2, rows)
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    ops.merge_candidates(to_dev(cand), width, out)
    got = to_host(out).view(np.uint32)
    # row 0: parts 1 and 3 tie at 2.0 -> part 1; row 1: parts 0, 1, 3 tie -> part 0; row 2: part 2; row 3: a part reported
    # a bad row; row 4: a non-finite value
    assert list(got) == [1000 + 10, 2, 2000 + 7, 0xFFFFFFFF, 0xFFFFFFFF]


def tiny_config(**kw):
    from inferrous_b200.qwen3 import Qwen3Config

    base = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=640, context=192)
    base.update(kw)
    return Qwen3Config(**base)


@pytest.mark.parametrize("batch,cfg", [
    (8, dict()),
    (5, dict(layers=3, hidden=1024, q_heads=8, kv_heads=2, intermediate=3072, vocab=4096, context=256)),
    (20, dict(layers=1, vocab=1024)),   # more rows than the fused head + selection takes: stored logits + select_token
])
def test_sequences_decoded_side_by_side_equal_sequences_decoded_alone(batch, cfg):
    """Ragged prompts (1 .. 150 tokens) decoded as one batch: every sequence's tokens, its final hidden row and its KV
    caches are bit-identical to the same sequence run through a batch of one, graph replay equals eager launches, the
    plain kernels (one thread per output, nothing fused) give the same bits, and the tokens are those of the
    single-request runner (whose attention kernel associates its sums differently)."""
    from inferrous_b200 import ops
    from inferrous_b200.qwen3 import Qwen3Runner, Qwen3Weights

    config = tiny_config(**cfg)
    weights = Qwen3Weights.random(config, seed=11)
    rng = np.random.default_rng(batch)
    lengths = [int(n) for n in rng.integers(1, 150, batch)]
    lengths[0], lengths[-1] = 1, 150
    prompts = [[int(t) for t in rng.integers(0, config.vocab, n)] for n in lengths]
    steps = 9
    side = Qwen3Runner(weights, batch=batch)
    tokens, _ = side.generate_batch(prompts, steps, use_graph=True)
    hidden = to_host(side.batch_ws.hidden).copy()
    eager, _ = side.generate_batch(prompts, steps, use_graph=False)
    assert eager == tokens and np.array_equal(to_host(side.batch_ws.hidden), hidden)
    plain = Qwen3Runner(weights, batch=batch, unfused=True)
    assert plain.generate_batch(prompts, steps)[0] == tokens
    assert np.array_equal(to_host(plain.batch_ws.hidden), hidden)
    alone = Qwen3Runner(weights, batch=1)
    alone._make_batch_buffers()
    classic = Qwen3Runner(weights)
    same_as_classic = 0
    for r, prompt in enumerate(prompts):
        one, _ = alone.generate_batch([prompt], steps)
        assert one[0] == tokens[r], r
        assert np.array_equal(to_host(alone.batch_ws.hidden)[0], hidden[r]), r
        n = lengths[r] + steps - 1
        for layer in range(config.layers):
            assert np.array_equal(to_host(alone.k_cache_all[layer][0, :n]), to_host(side.k_cache_all[layer][r, :n]))
            assert np.array_equal(to_host(alone.v_cache_all[layer][0, :n]), to_host(side.v_cache_all[layer][r, :n]))
        if r < 3:
            same_as_classic += classic.generate(prompt, steps)[0] == tokens[r]
    assert same_as_classic == 3
    assert ops.device_status() == (0, 0)


def test_attention_batched_more_rows_than_one_launch_takes(ops):
    """A batch beyond the row limit of one launch is cut into several launches inside the entry point: every row still
    equals the row computed in a smaller batch."""
    import torch

    rng = np.random.default_rng(300)
    rows, qh, kvh, capacity = 300, 4, 2, 256
    _, _, kc, vc = random_caches(rng, rows, capacity, kvh)
    qd = to_dev(oracle.bf16(rng.standard_normal((rows, qh * 128)).astype(np.float32)), "bf16")
    pos = to_dev(rng.integers(0, capacity, rows).astype(np.uint32))
    out = torch.full((rows, qh * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.attention_batched(qd, qh, kvh, kc, vc, pos, out, ops.attention_batched_workspace(rows, qh, kvh))
    for a, b in [(0, 150), (150, 300)]:
        part = torch.full((b - a, qh * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.attention_batched(qd[a:b], qh, kvh, kc[a:b], vc[a:b], pos[a:b], part, ops.attention_batched_workspace(b - a, qh, kvh))
        assert np.array_equal(to_host(part), to_host(out[a:b]))
    assert not np.isnan(to_host(out)).any()
    assert ops.device_status() == (0, 0)
