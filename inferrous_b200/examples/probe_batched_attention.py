"""Times qwen3_attention_batched alone on a ragged batch (the attention launch of one layer of a batched decode step):
`rows` sequences whose context lengths are drawn uniformly from [128, 4096], Qwen3-8B head counts by default.

    python -m inferrous_b200.examples.probe_batched_attention [q_heads kv_heads [rows]]

Prints one JSON line: microseconds per launch (CUDA events around 20 back-to-back launches; the caches of 64 sequences
are 1 GB, far beyond the L2) and the rate at which the visible keys and values stream."""
import json
import sys

import numpy as np
import torch

from inferrous_b200 import ops


def main() -> None:
    ops.init()
    qh = int(sys.argv[1]) if len(sys.argv) > 1 else 32
    kvh = int(sys.argv[2]) if len(sys.argv) > 2 else 8
    rows = int(sys.argv[3]) if len(sys.argv) > 3 else 64
    capacity = 4096
    rng = np.random.default_rng(4)
    contexts = rng.integers(128, capacity + 1, rows)
    k_cache = torch.randn(rows, capacity, kvh, 128, device="cuda", dtype=torch.bfloat16)
    v_cache = torch.randn(rows, capacity, kvh, 128, device="cuda", dtype=torch.bfloat16)
    q = torch.randn(rows, qh * 128, device="cuda", dtype=torch.bfloat16)
    positions = torch.tensor((contexts - 1).astype(np.int32), device="cuda")
    out = torch.empty(rows, qh * 128, device="cuda", dtype=torch.bfloat16)
    workspace = ops.attention_batched_workspace(rows, qh, kvh)
    for _ in range(3):
        ops.attention_batched(q, qh, kvh, k_cache, v_cache, positions, out, workspace)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 20
    start.record()
    for _ in range(launches):
        ops.attention_batched(q, qh, kvh, k_cache, v_cache, positions, out, workspace)
    stop.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(stop) * 1e3 / launches
    nbytes = int(contexts.sum()) * kvh * 128 * 2 * 2
    print(json.dumps({"rows": rows, "q_heads": qh, "kv_heads": kvh, "us_per_launch": round(us, 1), "kv_MB": round(nbytes / 1e6, 1),
                      "GB/s": round(nbytes / us / 1e3, 1), "device_status": ops.device_status()}))


if __name__ == "__main__":
    main()
