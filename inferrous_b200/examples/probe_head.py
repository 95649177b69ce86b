"""The two output heads on one row against the Qwen3 vocabulary, timed launch by launch: the reference's bf16 head
(`qwen3_head_bf16`, its summation order, greedy selection fused in) and the W8A8 head (`w8a8_linear_argmax`).

    python -m inferrous_b200.examples.probe_head

Random weights; every launch after a 256 MB read that displaces the L2; prints the median time of five launches and
the weight bytes per second."""
import statistics

import torch

from inferrous_b200 import ops


def main() -> None:
    ops.init()
    vocab, hidden = 151936, 4096
    gen = torch.Generator(device="cuda").manual_seed(2)
    w_bf16 = torch.empty((vocab, hidden), dtype=torch.bfloat16, device="cuda").normal_(0.0, 0.02, generator=gen)
    x = torch.randn((1, hidden), device="cuda", generator=gen).to(torch.bfloat16)
    w_i8 = torch.randint(-127, 128, (vocab, hidden), dtype=torch.int8, device="cuda", generator=gen)
    scale = ((0.5 + torch.rand(vocab, device="cuda", generator=gen)) / 4000.0).float()
    matrix = ops.Matrix(w_i8, scale)
    q = torch.randint(-127, 128, (1, hidden), dtype=torch.int8, device="cuda", generator=gen)
    a = torch.full((1,), 0.01, dtype=torch.float32, device="cuda")
    token = torch.zeros(1, dtype=torch.int32, device="cuda")
    flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")
    cases = [("head_bf16 + select_token", lambda: ops.head_bf16(x, w_bf16, token=token), 2 * vocab * hidden),
             ("W8A8 head + select_token", lambda: ops.linear_argmax(q, a, matrix, token), vocab * hidden)]
    for name, fn, nbytes in cases:
        times = []
        for _ in range(5):
            flush.sum()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            stop.record()
            stop.synchronize()
            times.append(start.elapsed_time(stop) * 1e3)
        us = statistics.median(times)
        print(f"{name}: {us:.1f} us, {nbytes / us / 1e3:.0f} GB/s of weights, token {int(token[0])}")
    if ops.device_status() != (0, 0):
        raise SystemExit("device status is not clean")


if __name__ == "__main__":
    main()
