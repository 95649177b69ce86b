"""The whole Qwen3-8B architecture at its real size (36 layers, hidden 4096, 32 query / 8 key-value heads, intermediate
12288, vocabulary 151936; random-init W8A8 weights), batch 1, a 129-token prompt of uniform-random token ids followed
by 128 greedy decode steps: the fast path (tensor-core prefill, fused decode kernels, fused head + selection, the
decode step replayed as a CUDA graph with programmatic launches) against the same generation with the
one-thread-per-output projection and every fused step unfused.

This is the library's form of the reference's `reused_graphs_match_eager` (src/gpu.rs:945-982: graph replay against
eager launches, tokens and logit hashes equal) and of its per-run regression check (tools/check_regression.py:10-27:
every token id and logit hash equal to the unoptimized implementation's).  int32 sums are exact and the epilogue is
element-wise IEEE arithmetic, so the two generations must agree bit for bit: token ids, the final hidden row and every
KV-cache entry -- the logit divergence between them is zero by construction."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_qwen3_8b_129_plus_128_fast_equals_plain():
    import torch

    from inferrous_b200 import ops
    from inferrous_b200.qwen3 import Qwen3Config, Qwen3Runner, Qwen3Weights

    free, _ = torch.cuda.mem_get_info()
    if free < 40 << 30:
        pytest.skip("needs 40 GB of free device memory")
    config = Qwen3Config.qwen3_8b()
    weights = Qwen3Weights.random(config, seed=3)
    rng = np.random.default_rng(129)
    prompt = [int(t) for t in rng.integers(0, config.vocab, 129)]
    steps = 128
    fast = Qwen3Runner(weights)
    tokens_fast, _ = fast.generate(prompt, steps, use_graph=True)
    plain = Qwen3Runner(weights, unfused=True)
    tokens_plain, _ = plain.generate(prompt, steps)
    assert len(tokens_fast) == steps and all(0 <= t < config.vocab for t in tokens_fast)
    assert tokens_fast == tokens_plain
    assert len(set(tokens_fast)) > 8  # not a degenerate generation
    assert torch.equal(fast.decode.hidden, plain.decode.hidden)
    n = len(prompt) + steps - 1
    for layer in range(config.layers):
        assert torch.equal(fast.k_cache[layer][:n], plain.k_cache[layer][:n]), layer
        assert torch.equal(fast.v_cache[layer][:n], plain.v_cache[layer][:n]), layer
    # eager launches of the fast kernels: the same tokens again (graph replay changes nothing)
    tokens_eager, _ = fast.generate(prompt, 24, use_graph=False)
    assert tokens_eager == tokens_fast[:24]
    assert ops.device_status() == (0, 0)
    del fast, plain, weights
    torch.cuda.empty_cache()
