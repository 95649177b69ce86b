"""Where the time of one resident decode step goes: per-layer step durations from the kernel's own cycle trace.

    python -m inferrous_b200.examples.trace_decode --prompt 129 --tokens 16

creates the decode plan with W8A8_DECODE_TRACE=1, generates a few tokens with random-init weights of the Qwen3-8B
architecture and prints, for the last step, the mean / minimum / maximum over the CTAs of every segment between two
trace points (averaged over the layers, first and last left out), in microseconds at the sampled SM clock.

Tensor parallel: launched under torchrun, every rank runs the kernel on its shard and rank 0 prints its own trace; the
segments that end at "exchange" are the waits for the other ranks' partial outputs of O and down:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m inferrous_b200.examples.trace_decode
"""
from __future__ import annotations

import argparse
import os

import numpy as np

POINTS = ["start", "norm1+quantize", "Q|K|V", "(requests)", "barrier", "attention", "barrier", "quantize", "O", "barrier",
          "norm2+quantize", "gate|up", "barrier", "quantize", "down", "barrier"]
POINTS_TP = POINTS[:9] + ["exchange"] + POINTS[10:15] + ["exchange"]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--prompt", type=int, default=129)
    ap.add_argument("--tokens", type=int, default=16)
    args = ap.parse_args()
    os.environ["W8A8_DECODE_TRACE"] = "1"

    import pynvml
    import torch

    from inferrous_b200 import ops
    from inferrous_b200.qwen3 import Qwen3Config, Qwen3Runner, Qwen3Weights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, group = 0, None
    if world > 1:
        import torch.distributed as dist

        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        rank, group = dist.get_rank(), dist.group.WORLD
    ops.init()
    config = Qwen3Config(layers=args.layers)
    weights = Qwen3Weights.random(config, seed=0).shard(rank, world)
    torch.cuda.empty_cache()
    runner = Qwen3Runner(weights, group=group, resident=True)
    if runner.plan is None:
        raise SystemExit("the resident decode kernel does not support this shape or device")
    prompt = [int(t) for t in np.random.default_rng(0).integers(0, config.vocab, args.prompt)]
    runner.generate(prompt, args.tokens)
    _, seconds = runner.generate(prompt, args.tokens)
    if world > 1:
        slowest = torch.tensor(seconds, dtype=torch.float64, device="cuda")
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        seconds = slowest.tolist()
        if rank != 0:
            torch.cuda.synchronize()
            dist.barrier()
            os._exit(0)  # captured graphs hold NCCL work: skip the communicator teardown
    pynvml.nvmlInit()
    mhz = float(pynvml.nvmlDeviceGetClockInfo(pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device()), pynvml.NVML_CLOCK_SM))
    print(f"host-visible ms per token (median): {float(np.median(seconds[1:])) * 1e3:.4f}; SM clock {mhz:.0f} MHz")
    t = runner.plan.trace().astype(np.float64)          # [ctas, layers, points]
    inner = slice(1, max(2, config.layers - 1))
    d = np.diff(t, axis=2)[:, inner, :] / mhz            # us
    names = POINTS_TP if world > 1 else POINTS
    print(f"{'segment ending at':24s} {'mean':>8s} {'min CTA':>8s} {'max CTA':>8s}" + (f"   (rank 0 of {world})" if world > 1 else ""))
    total = 0.0
    for i in range(d.shape[2]):
        per_cta = d[:, :, i].mean(axis=1)
        total += per_cta.mean()
        print(f"{names[i + 1]:24s} {per_cta.mean():8.2f} {per_cta.min():8.2f} {per_cta.max():8.2f}")
    print(f"per layer: {total:.2f} us; whole kernel (CTA 0): {(t[0, -1, -2] - t[0, 0, 0]) / mhz:.1f} us")
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
