"""Times the three activation quantizers at prefill size (4096 rows): plain (K = 4096), fused with RMSNorm (K = 4096) and
fused with SwiGLU ([4096, 24576] -> [4096, 12288]), each as the median of three launches with the L2 displaced by a
256 MB read before every launch.

    python -m inferrous_b200.examples.probe_quantizers

Prints one line per kernel: microseconds and algorithmic GB/s (2MK in + MK out; SwiGLU reads 4MI)."""
import statistics

import torch

from inferrous_b200 import ops


def activations(rows: int, width: int, seed: int) -> torch.Tensor:
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((rows, width), generator=gen, device="cuda", dtype=torch.float32)
    x[:, torch.randperm(width, generator=gen, device="cuda")[:8]] *= 20.0  # eight outlier channels
    return x.to(torch.bfloat16)


def main() -> None:
    ops.init()
    M, K, I = 4096, 4096, 12288
    x, gate_up = activations(M, K, 1), activations(M, 2 * I, 2)
    gamma = (1.0 + 0.1 * torch.randn(K, device="cuda")).to(torch.bfloat16)
    q4 = torch.empty((M, K), dtype=torch.int8, device="cuda")
    q12 = torch.empty((M, I), dtype=torch.int8, device="cuda")
    scale = torch.empty((M,), dtype=torch.float32, device="cuda")
    flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")
    cases = [("quantize", lambda: ops.quantize(x, q4, scale), 3 * M * K),
             ("rmsnorm_quantize", lambda: ops.norm_quantize(x, gamma, None, q4, scale, None), 3 * M * K),
             ("swiglu_quantize", lambda: ops.swiglu_quantize(gate_up[:, :I], gate_up[:, I:], q12, scale), 5 * M * I)]
    for name, fn, nbytes in cases:
        times = []
        for _ in range(3):
            flush.sum()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            stop.record()
            stop.synchronize()
            times.append(start.elapsed_time(stop) * 1e3)
        us = statistics.median(times)
        print(f"{name}: {us:.1f} us, {nbytes / us / 1e3:.0f} GB/s")


if __name__ == "__main__":
    main()
