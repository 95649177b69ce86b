"""One projection of the Qwen3-8B shape set through `w8a8_linear`, timed launch by launch: a small driver for profiling.

    python -m inferrous_b200.examples.probe_linear --shape down --tokens 64                 # the variant the library picks
    python -m inferrous_b200.examples.probe_linear --shape qkv --tokens 4096 --variant 8    # a forced variant (w8a8.h)

Random int8 weights and activation codes; `--launches` launches, each after a 256 MB read that displaces the L2; prints the
median time, TOPS and algorithmic GB/s (N K + 4 N + M K + 4 M + 2 M N bytes), and checks the output against the
one-thread-per-output kernel once."""
import argparse
import statistics

import torch

from inferrous_b200 import capi, ops

SHAPES = {"qkv": (4096, 6144), "o": (4096, 4096), "gate_up": (4096, 24576), "down": (12288, 4096), "lm_head": (4096, 151936)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", choices=sorted(SHAPES), default="down")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--variant", type=int, default=capi.VARIANT_AUTO)
    ap.add_argument("--launches", type=int, default=5)
    args = ap.parse_args()
    ops.init()
    K, N = SHAPES[args.shape]
    M = args.tokens
    gen = torch.Generator(device="cuda").manual_seed(1)
    w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=gen)
    scale = ((0.5 + torch.rand(N, device="cuda", generator=gen)) / 4000.0).float()
    matrix = ops.Matrix(w, scale)
    q = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=gen)
    a = (0.01 + 0.01 * torch.rand(M, device="cuda", generator=gen)).float()
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    if M * N <= 1 << 26:  # the plain kernel is slow: keep the check to sizes it finishes in a second or so
        expect = torch.empty_like(y)
        ops.linear_quantized(q, a, matrix, expect, capi.VARIANT_NAIVE)
        ops.linear_quantized(q, a, matrix, y, args.variant)
        if not torch.equal(y.view(torch.int16), expect.view(torch.int16)):
            raise SystemExit("output differs from the one-thread-per-output kernel")
    flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")
    times = []
    for _ in range(args.launches):
        flush.sum()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        ops.linear_quantized(q, a, matrix, y, args.variant)
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop) * 1e3)
    us = statistics.median(times)
    nbytes = N * K + 4 * N + M * K + 4 * M + 2 * M * N
    print(f"{args.shape} M={M} variant={args.variant}: {us:.1f} us, {2 * M * N * K / us / 1e6:.0f} TOPS, {nbytes / us / 1e3:.0f} GB/s")
    status = ops.device_status()
    if status != (0, 0):
        raise SystemExit(f"device status {status}")


if __name__ == "__main__":
    main()
