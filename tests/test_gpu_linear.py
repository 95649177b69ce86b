"""GPU parity of the W8A8 projection (INT8xINT8->INT32 product + dequantizing epilogue).
Mirrors the `linear` arm of independent_operators (src/conformance.rs:203-361: every kernel variant
must equal the fixture exactly) and fused_gate_up_matches_separate (:741-839).  INT32 accumulators
and bf16 outputs are compared bit for bit.  All calls go through the C ABI."""
import os

import numpy as np
import pytest

from oracle import oracle
from tests.util import bits, empty_act, synth_activations, synth_weights, to_dev, to_host

pytestmark = pytest.mark.gpu

NAIVE, DP4A, MMA, TC, SKINNY, PAIR, CLUSTER = 1, 2, 3, 4, 5, 8, 9
CARRIERS = ["bf16", "f32"]


@pytest.fixture(scope="module")
def ops():
    import torch
    from inferrous_b200 import ops as o

    assert torch.cuda.is_available()
    o.init()
    return o


def variants_for(M):
    v = [NAIVE, TC, PAIR]
    if M <= 256:
        v.append(SKINNY)
    if M <= 256:
        v.append(CLUSTER)
    if os.environ.get("W8A8_TEST_SKIP_TCGEN05"):  # bring-up aid: check the SIMT variants alone
        v = [NAIVE]
    if M <= 4:
        v.append(DP4A)
    if M <= 64:
        v.append(MMA)
    return v


def check_status(ops):
    st, detail = ops.device_status()
    assert st == 0, f"device-side wait expired: detail {detail:#x}"


def make_matrix(ops, w, ws):
    return ops.Matrix(to_dev(w), to_dev(ws, "f32"))


def run_linear(ops, mat, q, asc, carrier, variant, residual=None):
    qd, ad = to_dev(q), to_dev(np.ascontiguousarray(asc, dtype=np.float32).reshape(-1), "f32")
    M, N = q.shape[0], mat.n
    y = empty_act((M, N), carrier)
    if residual is None:
        ops.linear_quantized(qd, ad, mat, y, variant)
        return to_host(y), None
    comb = empty_act((M, N), carrier)
    ops.linear_residual(qd, ad, mat, y, to_dev(residual, carrier), comb, variant)
    return to_host(y), to_host(comb)


def run_acc(ops, mat, q, variant):
    import torch

    acc = torch.full((q.shape[0], mat.n), 0x7FFFFFFF, dtype=torch.int32, device="cuda")
    ops.linear_acc_i32(to_dev(q), mat, acc, variant)
    return to_host(acc)


@pytest.mark.parametrize("carrier", CARRIERS)
def test_linear_fixtures_every_variant_exact(ops, fixtures, carrier):
    for c in fixtures.cases("linear"):
        q, w = fixtures.tensor(c, "q"), fixtures.tensor(c, "w")
        asc, ws = fixtures.tensor(c, "asc"), fixtures.tensor(c, "ws")
        expected = fixtures.tensor(c, "out")
        M, N = q.shape[0], w.shape[0]
        mat = make_matrix(ops, w, ws)
        acc_ref = oracle.linear_acc(q, w)
        # src/conformance.rs:220-225: residual operand ((i mod 17) - 8) * 0.0625
        res = (((np.arange(M * N) % 17) - 8) * 0.0625).astype(np.float32).reshape(M, N)
        comb_ref = oracle.residual(res, expected)
        for v in variants_for(M):
            y, _ = run_linear(ops, mat, q, asc, carrier, v)
            assert np.array_equal(bits(y), bits(expected)), (c["name"], v)
            y2, comb = run_linear(ops, mat, q, asc, carrier, v, residual=res)
            assert np.array_equal(bits(y2), bits(expected)), (c["name"], v, "y with residual")
            assert np.array_equal(bits(comb), bits(comb_ref)), (c["name"], v, "combined")
            assert np.array_equal(run_acc(ops, mat, q, v), acc_ref), (c["name"], v, "int32")
        # AUTO picks one of them
        y, _ = run_linear(ops, mat, q, asc, carrier, 0)
        assert np.array_equal(bits(y), bits(expected))
        check_status(ops)


def test_separate_residual_kernel_equals_fused(ops, fixtures):
    """`linear_residual` must equal `linear` followed by `residual` bitwise (src/conformance.rs:226-262)."""
    c = fixtures.cases("linear")[0]
    q, w, asc, ws = (fixtures.tensor(c, k) for k in ("q", "w", "asc", "ws"))
    mat = make_matrix(ops, w, ws)
    res = (((np.arange(33) % 17) - 8) * 0.0625).astype(np.float32).reshape(1, 33)
    y, comb = run_linear(ops, mat, q, asc, "f32", 0, residual=res)
    out = empty_act((1, 33), "f32")
    ops.residual(to_dev(res, "f32"), to_dev(y, "f32"), out)
    assert np.array_equal(bits(to_host(out)), bits(comb))


@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 8, 16])
def test_config0_and_decode_shapes_exact(ops, M):
    """M tokens x (K=4096 -> N=4096), the enlarged fixture shape: quantize on the GPU, then every variant
    against the CPU oracle: int8 codes, scales, int32 accumulators and bf16 outputs bit for bit."""
    import torch

    rng = np.random.default_rng(824 + M)
    K, N = 4096, 4096
    x = synth_activations(rng, M, K)
    w, ws = synth_weights(rng, N, K)
    mat = make_matrix(ops, w, ws)
    qd = torch.zeros((M, K), dtype=torch.int8, device="cuda")
    sd = torch.zeros((M,), dtype=torch.float32, device="cuda")
    ops.quantize(to_dev(x, "bf16"), qd, sd)
    q, s = oracle.quantize(x)
    assert np.array_equal(to_host(qd), q) and np.array_equal(bits(to_host(sd)), bits(s))
    acc_ref = oracle.linear_acc(q, w)
    y_ref = oracle.epilogue(acc_ref, s, ws)
    for v in variants_for(M) + [0]:
        y, _ = run_linear(ops, mat, q, s, "bf16", v)
        assert np.array_equal(bits(y), bits(y_ref)), v
        if v:
            assert np.array_equal(run_acc(ops, mat, q, v), acc_ref), v
    check_status(ops)


@pytest.mark.parametrize("M,K,N", [(1, 12288, 4096), (4, 4096, 6144), (16, 12288, 4096), (3, 128, 33), (4, 256, 8),
                                   (16, 4096, 1000), (33, 4096, 520), (64, 12288, 272)])
def test_ragged_shapes_exact(ops, M, K, N):
    rng = np.random.default_rng(M * 131 + N)
    q = rng.integers(-127, 128, (M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    q[0] = 127
    w[0] = 127
    w[N - 1] = -127
    asc = (rng.random(M, dtype=np.float32) / 64).astype(np.float32)
    ws = (rng.random(N, dtype=np.float32) / 64).astype(np.float32)
    mat = make_matrix(ops, w, ws)
    acc_ref = oracle.linear_acc(q, w)
    y_ref = oracle.epilogue(acc_ref, asc, ws)
    for v in variants_for(M):
        y, _ = run_linear(ops, mat, q, asc, "bf16", v)
        assert np.array_equal(bits(y), bits(y_ref)), v
        assert np.array_equal(run_acc(ops, mat, q, v), acc_ref), v
    check_status(ops)


@pytest.mark.parametrize("M", [1, 4, 16])
def test_grouped_qkv_equals_separate(ops, M):
    """`linear_triple`: Q, K, V in one launch == three separate projections (src/conformance.rs:263-300)."""
    rng = np.random.default_rng(5 + M)
    K = 4096
    q = rng.integers(-127, 128, (M, K), dtype=np.int8)
    asc = (rng.random(M, dtype=np.float32) / 64).astype(np.float32)
    mats, refs = [], []
    for N in (4096, 1024, 1024):
        w = rng.integers(-127, 128, (N, K), dtype=np.int8)
        ws = (rng.random(N, dtype=np.float32) / 64).astype(np.float32)
        mats.append(make_matrix(ops, w, ws))
        refs.append(oracle.linear(q, asc, w, ws))
    outs = [empty_act((M, m.n), "bf16") for m in mats]
    ops.linear_grouped(to_dev(q), to_dev(asc, "f32"), mats, outs)
    for o, r in zip(outs, refs):
        assert np.array_equal(bits(to_host(o)), bits(r))
    # a pair, with a ragged second matrix
    outs2 = [empty_act((M, m.n), "bf16") for m in mats[:2]]
    ops.linear_grouped(to_dev(q), to_dev(asc, "f32"), mats[:2], outs2)
    for o, r in zip(outs2, refs[:2]):
        assert np.array_equal(bits(to_host(o)), bits(r))


@pytest.mark.parametrize("K,N", [(128, 33), (4096, 12288)])
@pytest.mark.parametrize("M", [1, 3, 8])
def test_fused_gate_up_matches_separate(ops, K, N, M):
    """src/conformance.rs:741-839 with its closed-form inputs: fused gate/up + SwiGLU + absmax equals the
    separate projections followed by `swiglu`, bitwise on gate, up, act and the maximum."""
    i = np.arange(K, dtype=np.int64)
    q1 = ((i * 13 % 255) - 127).astype(np.int8)
    q = np.stack([np.roll(q1, m) for m in range(M)])
    j = np.arange(K * N, dtype=np.int64)
    w0 = ((j * 31 % 255) - 127).astype(np.int8).reshape(N, K)
    w1 = ((j * 17 % 251) - 125).astype(np.int8).reshape(N, K)
    asc = np.full(M, 0.002, dtype=np.float32)
    n = np.arange(N)
    s0 = (np.float32(0.0001) * ((n % 7 + 1).astype(np.float32))).astype(np.float32)
    s1 = (np.float32(0.0001) * ((n % 11 + 1).astype(np.float32))).astype(np.float32)
    m0, m1 = make_matrix(ops, w0, s0), make_matrix(ops, w1, s1)
    qd, ad = to_dev(q), to_dev(asc, "f32")
    floor_bits = np.float32(1e-8).view(np.uint32)
    # separate: two projections (naive variant) + swiglu
    g = empty_act((M, N), "f32")
    u = empty_act((M, N), "f32")
    ops.linear_quantized(qd, ad, m0, g, NAIVE)
    ops.linear_quantized(qd, ad, m1, u, NAIVE)
    assert np.array_equal(bits(to_host(g)), bits(oracle.linear(q, asc, w0, s0)))
    assert np.array_equal(bits(to_host(u)), bits(oracle.linear(q, asc, w1, s1)))
    act = empty_act((M, N), "f32")
    mx = to_dev(np.full(M, floor_bits, dtype=np.uint32))
    ops.swiglu(g, u, act, mx)
    # fused
    g2, u2, act2 = empty_act((M, N), "f32"), empty_act((M, N), "f32"), empty_act((M, N), "f32")
    mx2 = to_dev(np.full(M, floor_bits, dtype=np.uint32))
    ops.linear_swiglu(qd, ad, m0, m1, g2, u2, act2, mx2)
    assert np.array_equal(bits(to_host(g2)), bits(to_host(g))), "gate bits"
    assert np.array_equal(bits(to_host(u2)), bits(to_host(u))), "up bits"
    assert np.array_equal(bits(to_host(act2)), bits(to_host(act))), "activation bits"
    a = to_host(act)
    expect = np.maximum(np.abs(a).max(axis=1), np.float32(1e-8)).astype(np.float32).view(np.uint32)
    assert np.array_equal(to_host(mx2).view(np.uint32), expect), "activation maximum"
    assert np.array_equal(to_host(mx).view(np.uint32), expect)
    if M <= 4:  # gate/up outputs are optional in the fused decode kernel
        act3 = empty_act((M, N), "f32")
        ops.linear_swiglu(qd, ad, m0, m1, None, None, act3, None)
        assert np.array_equal(bits(to_host(act3)), bits(a))


@pytest.mark.parametrize("M,K,N", [(129, 4096, 4096), (512, 4096, 6144), (257, 12288, 4096), (130, 4096, 33), (64, 4096, 256),
                                   (1000, 4096, 1000), (17, 12288, 4096), (48, 4096, 24576), (256, 4096, 1024), (200, 128, 136)])
def test_prefill_shapes_exact(ops, M, K, N):
    """Tensor-core path against the CPU oracle at sizes the oracle finishes in seconds, with ragged M and N tails."""
    rng = np.random.default_rng(M + N)
    x = synth_activations(rng, M, K)
    w, ws = synth_weights(rng, N, K)
    q, s = oracle.quantize(x)
    mat = make_matrix(ops, w, ws)
    acc_ref = oracle.linear_acc(q, w)
    y_ref = oracle.epilogue(acc_ref, s, ws)
    for v in variants_for(M)[1:]:
        assert np.array_equal(run_acc(ops, mat, q, v), acc_ref), v
        yv, _ = run_linear(ops, mat, q, s, "f32", v)
        assert np.array_equal(bits(yv), bits(y_ref)), v
    y, _ = run_linear(ops, mat, q, s, "bf16", 0)
    assert np.array_equal(bits(y), bits(y_ref))
    res = oracle.bf16(rng.standard_normal((M, N), dtype=np.float32))
    for v in variants_for(M)[1:]:
        y2, comb = run_linear(ops, mat, q, s, "bf16", v, residual=res)
        assert np.array_equal(bits(y2), bits(y_ref)), v
        assert np.array_equal(bits(comb), bits(oracle.residual(res, y_ref))), v
    check_status(ops)


def test_bad_arguments_are_rejected(ops):
    import ctypes as C
    import torch
    from inferrous_b200 import capi

    lib = capi.load()
    w = torch.zeros((8, 100), dtype=torch.int8, device="cuda")
    s = torch.zeros((8,), dtype=torch.float32, device="cuda")
    h = C.c_void_p()
    assert lib.w8a8_weight_create(w.data_ptr(), s.data_ptr(), 8, 100, C.byref(h)) == 2  # K % 128
    assert lib.w8a8_weight_create(None, s.data_ptr(), 8, 128, C.byref(h)) == 1
    assert lib.w8a8_linear(None, None, None, 1, None, None, None, 0, None) == 1
    rng = np.random.default_rng(0)
    wq, ws = synth_weights(rng, 16, 128)
    mat = make_matrix(ops, wq, ws)
    q = torch.zeros((5, 128), dtype=torch.int8, device="cuda")
    a = torch.ones((5,), dtype=torch.float32, device="cuda")
    y = torch.zeros((5, 16), dtype=torch.bfloat16, device="cuda")
    # dp4a variant refuses M > 4
    assert lib.w8a8_linear_ex(q.data_ptr(), a.data_ptr(), mat.handle, 5, None, y.data_ptr(), None, 0, DP4A, None) == 3
    # residual without combined
    assert lib.w8a8_linear(q.data_ptr(), a.data_ptr(), mat.handle, 5, y.data_ptr(), y.data_ptr(), None, 0, None) == 1


def test_graph_replay_matches_eager(ops):
    """Every launch call is legal inside stream capture and a replayed graph reproduces the eager results bit for bit
    (operator-level counterpart of reused_graphs_match_eager, src/gpu.rs:945-982), with programmatic launches on."""
    import torch

    rng = np.random.default_rng(99)
    K, N, I = 4096, 4096, 12288
    w, ws = synth_weights(rng, N, K)
    mat = make_matrix(ops, w, ws)
    wg, wgs = synth_weights(rng, 256, K)
    wu, wus = synth_weights(rng, 256, K)
    mg, mu = make_matrix(ops, wg, wgs), make_matrix(ops, wu, wus)
    gamma = to_dev(oracle.bf16((1 + 0.1 * rng.standard_normal(K)).astype(np.float32)), "bf16")
    ops.set_programmatic_launch(True)
    try:
        for M in (1, 16, 129, 300):
            x = to_dev(synth_activations(rng, M, K), "bf16")
            res = to_dev(oracle.bf16(rng.standard_normal((M, N), dtype=np.float32)), "bf16")
            q = torch.zeros((M, K), dtype=torch.int8, device="cuda")
            s = torch.zeros((M,), dtype=torch.float32, device="cuda")
            y, comb = empty_act((M, N), "bf16"), empty_act((M, N), "bf16")
            act = empty_act((M, 256), "bf16")
            g, u = empty_act((M, 256), "bf16"), empty_act((M, 256), "bf16")
            mx = torch.zeros((M,), dtype=torch.int32, device="cuda")

            def chain():
                ops.norm_quantize(x, gamma, None, q, s, mx)
                ops.linear_residual(q, s, mat, y, res, comb)
                if M <= 16:
                    ops.linear_swiglu(q, s, mg, mu, g, u, act, mx)

            chain()
            torch.cuda.synchronize()
            outs = (q, s, y, comb, act, mx) if M <= 16 else (q, s, y, comb)
            eager = [t.clone() for t in outs]
            for t in outs:
                t.zero_()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                chain()
            for _ in range(2):
                mx.zero_()
                graph.replay()
            torch.cuda.synchronize()
            for a, b in zip(eager, outs):
                assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), M
    finally:
        ops.set_programmatic_launch(False)
    check_status(ops)


def test_tp_allreduce_single_rank_degenerate(ops):
    """w8a8_tp_allreduce with tp=1 (the only form one GPU can run): push to self, wait on self, out = bf16(partial),
    repeated so that both halves of the staging buffer and the device-side call counter are exercised."""
    import ctypes as C
    import torch
    from inferrous_b200 import capi

    lib = capi.load()
    slot = 16 * 4096
    buf = torch.zeros(2 * slot, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    seq = torch.zeros(4, dtype=torch.int32, device="cuda")
    bufs = (C.c_void_p * 1)(buf.data_ptr())
    fl = (C.c_void_p * 1)(flags.data_ptr())
    for call in range(5):
        n = (4096, 16 * 4096, 4 * 4096, 16 * 4096, 4096)[call]  # different sizes are cut into different CTA counts
        x = (torch.randn(n, device="cuda") * (call + 1)).to(torch.bfloat16)
        out = torch.zeros_like(x)
        st = lib.w8a8_tp_allreduce(x.data_ptr(), out.data_ptr(), n, 0, bufs, fl, seq.data_ptr(), 0, 1, slot, None)
        assert st == 0
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), x.view(torch.int16))
    assert seq.tolist() == [5, 0, 0, 0] and flags[0].item() == 5
    check_status(ops)
    # bad arguments
    assert lib.w8a8_tp_allreduce(x.data_ptr(), out.data_ptr(), n, 0, bufs, fl, seq.data_ptr(), 1, 1, slot, None) == 1
    assert lib.w8a8_tp_allreduce(x.data_ptr(), out.data_ptr(), n + 3, 0, bufs, fl, seq.data_ptr(), 0, 1, 2 * slot, None) == 2


def host_argmax(y):
    """model::argmax (src/model.rs:206-218): first index of the maximum; rows with a non-finite value are rejected."""
    out = []
    for row in y:
        out.append(0xFFFFFFFF if not np.all(np.isfinite(row)) else int(np.argmax(row)))  # np.argmax returns the first maximum
    return np.array(out, dtype=np.uint32)


@pytest.mark.parametrize("M,K,N", [(1, 4096, 151936), (4, 4096, 4096), (16, 128, 33), (9, 4096, 1000)])
def test_linear_argmax_matches_linear_then_select(ops, M, K, N):
    """Fused head + greedy selection == projection followed by the reference's selection rule, including ties
    (duplicated weight rows give equal logits: the lowest index must win) and the winning value."""
    import torch

    rng = np.random.default_rng(N + M)
    q = rng.integers(-127, 128, (M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (N, K), dtype=np.int8)
    ws = np.full(N, 1.0 / 4096, dtype=np.float32)
    # make the maximum appear several times: copy the best channel of token 0 to other places
    acc0 = (q[:1].astype(np.int64) @ w.astype(np.int64).T)[0]
    best = int(np.argmax(acc0))
    for dup in (N - 1, N // 2, max(0, best - 1)):
        w[dup] = w[best]
    asc = (rng.random(M, dtype=np.float32) / 64 + 1e-3).astype(np.float32)
    mat = make_matrix(ops, w, ws)
    y = empty_act((M, N), "f32")
    ops.linear_quantized(to_dev(q), to_dev(asc, "f32"), mat, y, NAIVE)
    expect = host_argmax(to_host(y))
    tok = torch.zeros(M, dtype=torch.int32, device="cuda")
    val = torch.zeros(M, dtype=torch.float32, device="cuda")
    for _ in range(2):  # the candidate buffer is reused
        ops.linear_argmax(to_dev(q), to_dev(asc, "f32"), mat, tok, val)
    got = to_host(tok).view(np.uint32)
    assert np.array_equal(got, expect)
    yh = to_host(y)
    assert np.array_equal(bits(to_host(val)), bits(yh[np.arange(M), expect.astype(np.int64)]))
    assert expect[0] == min(best, N - 1, N // 2, max(0, best - 1))  # the lowest of the equal maxima wins the tie


def test_linear_argmax_rejects_non_finite_rows(ops):
    import torch

    rng = np.random.default_rng(3)
    M, K, N = 3, 256, 64
    q = rng.integers(1, 128, (M, K), dtype=np.int8)
    w = rng.integers(1, 128, (N, K), dtype=np.int8)
    ws = np.full(N, 1e-3, dtype=np.float32)
    asc = np.array([1e-3, np.inf, 1e-3], dtype=np.float32)  # token 1 overflows to infinity everywhere
    mat = make_matrix(ops, w, ws)
    tok = torch.zeros(M, dtype=torch.int32, device="cuda")
    ops.linear_argmax(to_dev(q), to_dev(asc, "f32"), mat, tok, None)
    got = to_host(tok).view(np.uint32)
    y = oracle.linear(q, asc, w, ws)
    assert got[1] == 0xFFFFFFFF
    assert got[0] == np.argmax(y[0]) and got[2] == np.argmax(y[2])


@pytest.mark.parametrize("M", [1, 3, 4, 16, 40])
def test_fused_allreduce_with_one_rank_is_linear_residual(ops, M):
    """w8a8_linear_allreduce with a tensor-parallel group of one: the packets go to this GPU's own buffer, the consumer sums
    one contribution, and the result must be the single-GPU `linear_residual`, over several calls (both halves of the
    packet buffer, tags that keep growing)."""
    import ctypes as C

    import torch

    from inferrous_b200 import capi

    rng = np.random.default_rng(M)
    K, N = 512, 384
    w, ws = synth_weights(rng, N, K)
    mat = make_matrix(ops, w, ws)
    slot = 64 * N
    packets = torch.zeros(2 * slot * 2, dtype=torch.int32, device="cuda")
    seq = torch.zeros(4, dtype=torch.int32, device="cuda")
    peers = (C.c_void_p * 1)(packets.data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(5):
        q = to_dev(rng.integers(-127, 128, (M, K), dtype=np.int8))
        a = to_dev(rng.uniform(0.01, 0.02, M).astype(np.float32), "f32")
        res = to_dev(oracle.bf16(rng.standard_normal((M, N)).astype(np.float32)), "bf16")
        y_ref, c_ref = empty_act((M, N), "bf16"), empty_act((M, N), "bf16")
        ops.linear_residual(q, a, mat, y_ref, res, c_ref)
        y, comb = empty_act((M, N), "bf16"), empty_act((M, N), "bf16")
        capi.check(capi.load().w8a8_linear_allreduce(q.data_ptr(), a.data_ptr(), mat.handle, M, res.data_ptr(), y.data_ptr(),
                                                     comb.data_ptr(), 0, peers, seq.data_ptr(), 0, 1, slot, stream),
                   "w8a8_linear_allreduce")
        assert torch.equal(y.view(torch.int16), y_ref.view(torch.int16)), call
        assert torch.equal(comb.view(torch.int16), c_ref.view(torch.int16)), call
    assert int(seq[0]) == 5
    check_status(ops)


@pytest.mark.parametrize("bn", [256, 192, 128])
def test_pair_kernel_every_tile_width_exact(ops, bn, monkeypatch):
    """The CTA-pair kernel with 256, 192 and 128 output channels per tile (W8A8_PAIR_BN forces a width): partial tiles in
    both directions, residual epilogue, raw accumulators -- all equal to the one-thread-per-output kernel."""
    monkeypatch.setenv("W8A8_PAIR_BN", str(bn))
    rng = np.random.default_rng(bn)
    for M, K, N in [(300, 512, 1000), (129, 4096, 200), (512, 1024, 768)]:
        q = rng.integers(-127, 128, (M, K), dtype=np.int8)
        w = rng.integers(-127, 128, (N, K), dtype=np.int8)
        asc = (rng.random(M, dtype=np.float32) / 64).astype(np.float32)
        ws = (rng.random(N, dtype=np.float32) / 64).astype(np.float32)
        res = oracle.bf16(rng.standard_normal((M, N)).astype(np.float32))
        mat = make_matrix(ops, w, ws)
        y, comb = run_linear(ops, mat, q, asc, "bf16", PAIR, residual=res)
        y0, comb0 = run_linear(ops, mat, q, asc, "bf16", NAIVE, residual=res)
        assert np.array_equal(bits(y), bits(y0)) and np.array_equal(bits(comb), bits(comb0))
        assert np.array_equal(run_acc(ops, mat, q, PAIR), run_acc(ops, mat, q, NAIVE))
    check_status(ops)
