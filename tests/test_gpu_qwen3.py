"""A whole Qwen3 W8A8 generation through the C ABI (inferrous_b200.qwen3): the fast kernels against the plain
ones, the captured decode graph against eager launches, and the GPU against the CPU restatement."""
import numpy as np
import pytest

from tests.qwen3_oracle import OracleModel, export
from tests.util import to_host

pytestmark = pytest.mark.gpu


def tiny_config(**kw):
    from inferrous_b200.qwen3 import Qwen3Config

    base = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=640, context=64)
    base.update(kw)
    return Qwen3Config(**base)


def test_tiny_model_matches_cpu_restatement():
    """Prefill of 5 tokens and 6 decode steps: same tokens as the CPU forward, final hidden rows within the
    reference's whole-model gate (relative L2 <= 5 %, tools/reference.py).  The only arithmetic that differs
    between the two is exp() inside attention (ex2.approx on the GPU)."""
    from inferrous_b200.qwen3 import Qwen3Runner, Qwen3Weights, Workspace

    import torch

    config = tiny_config()
    weights = Qwen3Weights.random(config, seed=4)
    prompt = [3, 600, 17, 17, 255]
    cpu = OracleModel(export(weights))
    expected = cpu.generate(prompt, 7)
    runner = Qwen3Runner(weights)
    got, _ = runner.generate(prompt, 7)
    assert got == expected
    # hidden state after the prefill
    ws = Workspace(config, len(prompt))
    runner.control.zero_()
    runner.forward(ws, torch.tensor(prompt, dtype=torch.int32, device="cuda"))
    hidden_cpu, _ = OracleModel(export(weights)).forward(np.array(prompt, np.uint32), 0)
    hidden_gpu = to_host(ws.hidden)
    rel = np.sqrt(((hidden_gpu.astype(np.float64) - hidden_cpu) ** 2).sum() / (hidden_cpu.astype(np.float64) ** 2).sum())
    assert rel <= 0.05
    from inferrous_b200 import ops

    assert ops.device_status() == (0, 0)


@pytest.mark.parametrize("prompt_len,steps,cfg", [
    (5, 12, dict()),
    (129, 10, dict(layers=3, hidden=1024, q_heads=8, kv_heads=2, intermediate=3072, vocab=4096, context=192)),
])
def test_fast_kernels_change_nothing_in_a_generation(prompt_len, steps, cfg):
    """Fused / tensor-core / graph-replayed generation == the same generation with the one-thread-per-output
    projection and unfused SwiGLU, quantizer and selection: identical tokens and bit-identical final hidden row."""
    from inferrous_b200.qwen3 import Qwen3Runner, Qwen3Weights

    config = tiny_config(**cfg)
    weights = Qwen3Weights.random(config, seed=9)
    rng = np.random.default_rng(2)
    prompt = [int(t) for t in rng.integers(0, config.vocab, prompt_len)]
    fast = Qwen3Runner(weights)
    plain = Qwen3Runner(weights, unfused=True)
    tokens_graph, _ = fast.generate(prompt, steps, use_graph=True)
    hidden_graph = to_host(fast.decode.hidden).copy()
    tokens_plain, _ = plain.generate(prompt, steps)
    assert tokens_graph == tokens_plain
    assert np.array_equal(hidden_graph, to_host(plain.decode.hidden))
    tokens_eager, _ = fast.generate(prompt, steps, use_graph=False)
    assert tokens_eager == tokens_plain
    assert np.array_equal(to_host(fast.decode.hidden), hidden_graph)
    for kw in (dict(prefetch_down_at="none"), dict(prefetch_rows=64, prefetch_down_at="qwm", prefetch_o=True),
               dict(fold_attention_quantizer=True)):
        other = Qwen3Runner(weights, **kw)  # L2 prefetch hints on other launches, or none at all
        assert other.generate(prompt, steps)[0] == tokens_plain
    for fold in ("with_max", "all"):  # quantizers inside the projection kernels
        folded = Qwen3Runner(weights, fold_quantizers=fold)
        tokens_folded, _ = folded.generate(prompt, steps)
        assert tokens_folded == tokens_plain
        assert np.array_equal(to_host(folded.decode.hidden), hidden_graph)
    for cache_fast, cache_plain in zip(fast.k_cache + fast.v_cache, plain.k_cache + plain.v_cache):
        n = prompt_len + steps - 1
        assert np.array_equal(to_host(cache_fast[:n]), to_host(cache_plain[:n]))
    from inferrous_b200 import ops

    assert ops.device_status() == (0, 0)


def test_context_limit_is_enforced_on_the_host():
    from inferrous_b200.qwen3 import Qwen3Runner, Qwen3Weights

    config = tiny_config(layers=1, context=16)
    runner = Qwen3Runner(Qwen3Weights.random(config, seed=1))
    with pytest.raises(ValueError):
        runner.generate(list(range(10)), 7)
    with pytest.raises(ValueError):
        runner.generate([], 3)
