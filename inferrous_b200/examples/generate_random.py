"""Greedy generation with random-init weights of a Qwen3-shaped model: a small driver for profiling and smoke runs.

    python -m inferrous_b200.examples.generate_random --layers 2 --prompt 300 --tokens 4 --eager

prints the generated token ids and the host-visible milliseconds of every step (the first is the prefill).
With --batch B the model decodes B sequences side by side (ragged: prompt lengths drawn uniformly from --contexts LO,HI):

    python -m inferrous_b200.examples.generate_random --layers 2 --batch 64 --contexts 128,4000 --tokens 4 --eager
"""
from __future__ import annotations

import argparse

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--prompt", type=int, default=129, help="prompt length (random token ids)")
    ap.add_argument("--tokens", type=int, default=32, help="tokens to generate")
    ap.add_argument("--eager", action="store_true", help="launch every decode step eagerly instead of replaying the graph")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--separate", action="store_true", help="one launch per operator instead of the resident decode kernel")
    ap.add_argument("--batch", type=int, default=0, help="decode this many sequences side by side (batched decode)")
    ap.add_argument("--contexts", default="128,4000", help="with --batch: range of the prompt lengths, LO,HI")
    args = ap.parse_args()

    from inferrous_b200 import ops
    from inferrous_b200.qwen3 import Qwen3Config, Qwen3Runner, Qwen3Weights

    ops.init()
    config = Qwen3Config(layers=args.layers)
    rng = np.random.default_rng(args.seed)
    if args.batch:
        lo, hi = (int(v) for v in args.contexts.split(","))
        runner = Qwen3Runner(Qwen3Weights.random(config, seed=args.seed), batch=args.batch)
        prompts = [[int(t) for t in rng.integers(0, config.vocab, int(n))] for n in rng.integers(lo, hi + 1, args.batch)]
        tokens, seconds = runner.generate_batch(prompts, args.tokens, use_graph=not args.eager)
        print("first sequence's tokens:", " ".join(map(str, tokens[0])))
    else:
        runner = Qwen3Runner(Qwen3Weights.random(config, seed=args.seed), resident=not args.separate)
        prompt = [int(t) for t in rng.integers(0, config.vocab, args.prompt)]
        tokens, seconds = runner.generate(prompt, args.tokens, use_graph=not args.eager)
        print("tokens:", " ".join(map(str, tokens)))
    print("ms per step:", " ".join(f"{s * 1e3:.3f}" for s in seconds))
    status, detail = ops.device_status()
    if status:
        raise SystemExit(f"device status {status}, detail {detail:#x}")


if __name__ == "__main__":
    main()
