"""The resident decode kernel (qwen3_decode_layers: all layers of a one-token step in one cooperative kernel, grid-wide
barriers instead of launches) against the launch-per-operator path it replaces: same tokens, bit-identical hidden row and
KV caches, eagerly launched and replayed from a CUDA graph."""
import numpy as np
import pytest

from tests.util import to_host

pytestmark = pytest.mark.gpu


def config(**kw):
    from inferrous_b200.qwen3 import Qwen3Config

    base = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=640, context=64)
    base.update(kw)
    return Qwen3Config(**base)


CASES = [
    # one 4096-byte round per weight row everywhere; two key splits come into use at 65 keys
    (dict(context=128), 5, 90),
    # Qwen3-like proportions: grouped heads, K of the down projection in the single-round form, contexts that cross several
    # split boundaries (64-key granularity) while decoding
    (dict(layers=3, hidden=1024, q_heads=8, kv_heads=2, intermediate=3072, vocab=4096, context=320), 60, 200),
    # down projection rows of two and three 4096-byte rounds (intermediate 4608 and 8448), hidden rows shorter than a round
    (dict(layers=1, intermediate=4608, context=64), 3, 20),
    (dict(layers=1, intermediate=8448, context=64), 3, 20),
    # one key/value head for eight query heads; widths that are not multiples of the 512-byte warp slice
    (dict(layers=2, hidden=1152, q_heads=8, kv_heads=1, intermediate=2176, vocab=1000, context=96), 17, 60),
    # more keys than sixteen splits of 64: the units read their keys and values from the cache, not from the copies
    # in shared memory, and decoding crosses the step from 64- to 96-key splits (1024 keys)
    (dict(context=1100), 1000, 60),
]


@pytest.mark.parametrize("cfg,prompt_len,steps", CASES)
def test_resident_step_equals_separate_launches(cfg, prompt_len, steps):
    import torch

    from inferrous_b200 import ops
    from inferrous_b200.qwen3 import Qwen3Runner, Qwen3Weights

    c = config(**cfg)
    weights = Qwen3Weights.random(c, seed=11)
    rng = np.random.default_rng(prompt_len)
    prompt = [int(t) for t in rng.integers(0, c.vocab, prompt_len)]
    resident = Qwen3Runner(weights, resident=True)
    assert resident.plan is not None
    separate = Qwen3Runner(weights, resident=False)
    assert separate.plan is None
    expected, _ = separate.generate(prompt, steps, use_graph=False)
    assert len(set(expected)) > 2
    for use_graph in (False, True):
        got, _ = resident.generate(prompt, steps, use_graph=use_graph)
        assert got == expected, use_graph
        assert torch.equal(resident.decode.hidden, separate.decode.hidden)
        n = prompt_len + steps - 1
        for layer in range(c.layers):
            assert torch.equal(resident.k_cache[layer][:n], separate.k_cache[layer][:n]), layer
            assert torch.equal(resident.v_cache[layer][:n], separate.v_cache[layer][:n]), layer
    assert ops.device_status() == (0, 0)


def test_resident_step_on_fewer_ctas(monkeypatch):
    """The share of every projection per CTA and the attention units per CTA follow the grid size: the result does not."""
    from inferrous_b200.qwen3 import Qwen3Runner, Qwen3Weights

    c = config(layers=2, hidden=512, q_heads=4, kv_heads=2, intermediate=1024, vocab=900, context=200)
    weights = Qwen3Weights.random(c, seed=5)
    prompt = [7, 8, 9, 500]
    expected, _ = Qwen3Runner(weights, resident=False).generate(prompt, 150, use_graph=False)
    for ctas in (24, 61):  # 64 attention units on 48 / 122 half-CTAs: some halves take two units
        monkeypatch.setenv("W8A8_DECODE_CTAS", str(ctas))
        runner = Qwen3Runner(weights, resident=True)
        assert runner.plan is not None
        assert runner.generate(prompt, 150)[0] == expected


def test_unsupported_shapes_keep_the_separate_launches():
    from inferrous_b200.qwen3 import Qwen3Runner, Qwen3Weights

    c = config(layers=1, intermediate=12288 + 128, context=32)  # a down-projection row longer than three rounds
    weights = Qwen3Weights.random(c, seed=2)
    runner = Qwen3Runner(weights)
    assert runner.plan is None
    tokens, _ = runner.generate([1, 2, 3], 4)
    assert tokens == Qwen3Runner(weights, unfused=True).generate([1, 2, 3], 4)[0]


def test_plan_arguments_are_checked():
    import ctypes as C

    import torch

    from inferrous_b200 import capi, ops
    from inferrous_b200.qwen3 import Qwen3Weights

    c = config(layers=1)
    weights = Qwen3Weights.random(c, seed=2)
    k = [torch.zeros(c.context, 1, 128, dtype=torch.bfloat16, device="cuda")]
    with pytest.raises(capi.W8A8Error) as bad:   # O's shape does not fit 3 query heads
        ops.DecodePlan(weights.layers, k, k, c.hidden, 3, 1, c.intermediate, c.eps, weights.rope)
    assert bad.value.status == 1
    lib = capi.load()
    out = C.c_void_p()
    assert lib.qwen3_decode_plan_create(None, 1, 256, 4, 2, 512, 64, 1e-6, None, 0, C.byref(out)) == 1
    assert lib.qwen3_decode_layers(None, None, None, None) == 1
    assert lib.qwen3_decode_plan_destroy(None) == 0


def test_cycle_trace_of_the_last_step(monkeypatch):
    """W8A8_DECODE_TRACE=1 at plan creation: every CTA notes its cycle counter at the boundaries of each layer's steps; the
    counts rise along a layer and from layer to layer, and the tokens are those of the kernel without marks."""
    from inferrous_b200 import capi
    from inferrous_b200.qwen3 import Qwen3Runner, Qwen3Weights

    c = config(layers=3, context=96)
    weights = Qwen3Weights.random(c, seed=8)
    prompt = [5, 6, 7]
    plain = Qwen3Runner(weights, resident=True)
    expected, _ = plain.generate(prompt, 20)
    with pytest.raises(capi.W8A8Error) as none:
        plain.plan.trace()
    assert none.value.status == 3
    monkeypatch.setenv("W8A8_DECODE_TRACE", "1")
    traced = Qwen3Runner(weights, resident=True)
    assert traced.generate(prompt, 20)[0] == expected
    t = traced.plan.trace()
    assert t.shape[1] == 3 and t.shape[2] == 16 and (t > 0).all()
    flat = t.reshape(t.shape[0], -1)
    assert (np.diff(flat, axis=1) >= 0).all()


@pytest.mark.parametrize("sliced", [0, 1])
@pytest.mark.parametrize("cfg,prompt_len,steps", [CASES[1], CASES[3]])
def test_resident_step_with_the_exchange_as_a_group_of_one(cfg, prompt_len, steps, sliced, monkeypatch):
    """The tensor-parallel form of the kernel (partial outputs of O and down sent as tagged packets, summed over the ranks
    in the next prologue, hidden and residual rows kept in shared memory) run on one GPU with itself as the only rank:
    the sum over one rank is the value itself, so the result must equal the single-GPU kernels' bit for bit.  sliced = 1:
    the form used from four ranks on (a CTA sums its slice of the row, a barrier, everyone reads the summed row)."""
    import torch

    monkeypatch.setenv("W8A8_DECODE_SLICED", str(sliced))

    from inferrous_b200 import ops
    from inferrous_b200.qwen3 import Qwen3Runner, Qwen3Weights

    c = config(**cfg)
    weights = Qwen3Weights.random(c, seed=13)
    prompt = [int(t) for t in np.random.default_rng(1).integers(0, c.vocab, prompt_len)]
    separate = Qwen3Runner(weights, resident=False)
    expected, _ = separate.generate(prompt, steps, use_graph=False)
    runner = Qwen3Runner(weights, resident=True, resident_exchange=True)
    assert runner.plan is not None and runner._exchange is not None
    for use_graph in (False, True):
        assert runner.generate(prompt, steps, use_graph=use_graph)[0] == expected
        assert torch.equal(runner.decode.hidden, separate.decode.hidden)
        n = prompt_len + steps - 1
        for layer in range(c.layers):
            assert torch.equal(runner.k_cache[layer][:n], separate.k_cache[layer][:n]), layer
    assert ops.device_status() == (0, 0)
