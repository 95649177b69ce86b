"""Tensor-parallel plumbing on CPU: two gloo ranks, each holding its shard, the CPU oracle standing in for the
kernels.  Column-split projections must reproduce the single-rank result bit for bit; row-split projections
(local absmax per K slice + summed partial outputs) must equal the same sharded arithmetic done in one process
and stay close to the unsharded result."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist

    from inferrous_b200 import tp
    from oracle import oracle

    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(11)  # same tensors on every rank
    M = 5
    results = {}
    for name, K, N in [("qkv", 256, 96), ("o", 512, 64), ("down", 1024, 32)]:
        x = oracle.bf16(rng.standard_normal((M, K), dtype=np.float32))
        w = rng.integers(-127, 128, (N, K), dtype=np.int8)
        ws = (rng.random(N, dtype=np.float32) / 64).astype(np.float32)
        xs = np.ascontiguousarray(tp.shard_activation(name, x, rank, world))
        wsh, wss = tp.shard_weight(name, w, ws, rank, world)
        q, s = oracle.quantize(xs)
        y = oracle.linear(q, s, np.ascontiguousarray(wsh), np.ascontiguousarray(wss))
        t = torch.from_numpy(y.copy())
        if tp.needs_all_reduce(name, world):
            tp.all_reduce_sum(t)
            results[name] = t.numpy()
        else:
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            results[name] = np.concatenate([p.numpy() for p in parts], axis=1)
    dist.barrier()
    if rank == 0:
        np.savez(Path(out_dir) / "tp.npz", **results)
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_linear(tmp_path):
    import torch.multiprocessing as mp

    from inferrous_b200 import tp
    from oracle import oracle

    port = 29500 + (os.getpid() % 2000)
    mp.start_processes(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    got = np.load(tmp_path / "tp.npz")
    rng = np.random.default_rng(11)
    M = 5
    for name, K, N in [("qkv", 256, 96), ("o", 512, 64), ("down", 1024, 32)]:
        x = oracle.bf16(rng.standard_normal((M, K), dtype=np.float32))
        w = rng.integers(-127, 128, (N, K), dtype=np.int8)
        ws = (rng.random(N, dtype=np.float32) / 64).astype(np.float32)
        q, s = oracle.quantize(x)
        full = oracle.linear(q, s, w, ws)
        if name in tp.ROW_SPLIT:
            k = K // 2
            parts = []
            for r in range(2):
                qr, sr = oracle.quantize(np.ascontiguousarray(x[:, r * k:(r + 1) * k]))
                parts.append(oracle.linear(qr, sr, np.ascontiguousarray(w[:, r * k:(r + 1) * k]), ws))
            assert np.array_equal(got[name], parts[0] + parts[1])  # the collective sums exactly these partials
            denom = np.linalg.norm(full)
            assert np.linalg.norm(got[name] - full) / denom < 0.02  # finer quantization, not the same numbers
        else:
            assert np.array_equal(got[name].view(np.uint32), full.view(np.uint32))


def test_shard_shapes():
    from inferrous_b200 import tp

    assert tp.shard_shape("qkv", 4096, 6144, 8) == (4096, 768)
    assert tp.shard_shape("gate_up", 4096, 24576, 4) == (4096, 6144)
    assert tp.shard_shape("o", 4096, 4096, 8) == (512, 4096)
    assert tp.shard_shape("down", 12288, 4096, 8) == (1536, 4096)
    assert tp.shard_shape("lm_head", 4096, 151936, 8) == (4096, 18992)
    assert tp.shard_shape("o", 4096, 4096, 1) == (4096, 4096)
    with pytest.raises(ValueError):
        tp.shard_shape("qkv", 4096, 6144, 5)
    assert tp.needs_all_reduce("down", 2) and not tp.needs_all_reduce("qkv", 2) and not tp.needs_all_reduce("down", 1)
