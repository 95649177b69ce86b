"""One rank of a tensor-parallel generation check; launched by torch.distributed.run from tests/test_gpu_tp_model.py.

Every rank builds the same random model (same seed), keeps its shard, and generates greedily in lockstep; rank 0 also
runs the unsharded model.  Rank 0 prints one JSON line: the tokens of both, and how far the tensor-parallel logits of
the prompt's last position are from the single-GPU ones (tensor parallelism rounds the partial outputs of O and down to
bf16 before they are summed, so the two are close, not identical)."""
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, tp = dist.get_rank(), dist.get_world_size()

    from inferrous_b200 import ops
    from inferrous_b200.qwen3 import Qwen3Config, Qwen3Runner, Qwen3Weights, Workspace

    ops.init()
    config = Qwen3Config(layers=2, hidden=512, q_heads=4, kv_heads=2, intermediate=1024, vocab=1024, context=192)
    full = Qwen3Weights.random(config, seed=21)
    shard = full.shard(rank, tp)
    prompt = [int(t) for t in np.random.default_rng(3).integers(0, config.vocab, int(sys.argv[1]))]
    steps = int(sys.argv[2])
    group = dist.group.WORLD

    # the decode step as one resident kernel per rank, the partial outputs of O and down exchanged as packets inside it
    resident = Qwen3Runner(shard, group=group)
    tokens_tp, _ = resident.generate(prompt, steps)
    hidden_resident = resident.decode.hidden.clone()
    tokens_eager, _ = Qwen3Runner(shard, group=group).generate(prompt, steps, use_graph=False)
    # the same step as one launch per operator, O and down with the all-reduce fused into the projection: same bits
    launches = Qwen3Runner(shard, group=group, resident=False)
    tokens_launches, _ = launches.generate(prompt, steps)
    resident_exact = resident.plan is not None and launches.plan is None and bool(torch.equal(hidden_resident, launches.decode.hidden))
    tokens_nccl, _ = Qwen3Runner(shard, group=group, fused_allreduce=False).generate(prompt, steps)

    # the fused projection + all-reduce against projection, gathered partials and a sum in rank order, bit for bit
    from inferrous_b200.tp import PeerLinear

    fused_exact = True
    peer = PeerLinear(group, 16 * 512)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    w = torch.randint(-127, 128, (512, 256), dtype=torch.int8, device="cuda", generator=gen)
    ws = (0.5 + torch.rand(512, device="cuda", generator=gen)) / 2000.0
    mat = ops.Matrix(w, ws.float())
    for call, rows in enumerate([1, 4, 16, 1, 3, 16, 2]):
        q = torch.randint(-127, 128, (rows, 256), dtype=torch.int8, device="cuda", generator=gen)
        a = 0.01 + torch.rand(rows, device="cuda", generator=gen) * 0.01
        res = torch.randn(rows, 512, device="cuda", generator=torch.Generator(device="cuda").manual_seed(call)).to(torch.bfloat16)
        y = torch.empty(rows, 512, dtype=torch.bfloat16, device="cuda")
        comb = torch.empty_like(y)
        peer.linear_residual(q, a.float(), mat, y, res, comb)
        part = torch.empty_like(y)
        ops.linear_quantized(q, a.float(), mat, part)
        parts = [torch.empty_like(part) for _ in range(tp)]
        dist.all_gather(parts, part)
        total = torch.zeros(rows, 512, dtype=torch.float32, device="cuda")
        for p in parts:
            total = total + p.float()
        expect = total.to(torch.bfloat16)
        fused_exact &= bool(torch.equal(y, expect)) and bool(torch.equal(comb, (res.float() + expect.float()).to(torch.bfloat16)))

    # batched decode under tensor parallelism: ragged sequences side by side; graph replay == eager launches, the fused
    # exchange == NCCL + residual on this model, and (fused exchange: partial outputs are exact per row and summed in
    # rank order) every sequence gives the tokens it gives when decoded alone
    rng = np.random.default_rng(17)
    prompts = [[int(t) for t in rng.integers(0, config.vocab, n)] for n in (1, 37, 150, 64, 9)]
    side = Qwen3Runner(shard, group=group, batch=len(prompts))
    batch_tokens, _ = side.generate_batch(prompts, steps)
    batch_eager, _ = side.generate_batch(prompts, steps, use_graph=False)
    batch_nccl, _ = Qwen3Runner(shard, group=group, batch=len(prompts), fused_allreduce=False).generate_batch(prompts, steps)
    alone = Qwen3Runner(shard, group=group, batch=1)
    alone._make_batch_buffers()
    batch_alone = [alone.generate_batch([p], steps)[0][0] for p in prompts]

    def prompt_logits(weights, grp):
        runner = Qwen3Runner(weights, unfused=True, group=grp)
        ws = Workspace(weights.config, len(prompt))
        runner.control.zero_()
        runner.forward(ws, torch.tensor(prompt, dtype=torch.int32, device="cuda"))
        torch.cuda.synchronize()
        return runner.logits[0].float().cpu().numpy()

    logits_tp = prompt_logits(shard, group)
    result = {"rank": rank, "tp": tp, "tokens_tp": tokens_tp, "tokens_tp_eager": tokens_eager, "tokens_nccl": tokens_nccl,
              "fused_exact": fused_exact, "tokens_launches": tokens_launches, "resident_exact": resident_exact, "batch_tokens": batch_tokens, "batch_eager": batch_eager, "batch_nccl": batch_nccl,
              "batch_alone": batch_alone}
    if rank == 0:
        tokens_single, _ = Qwen3Runner(full).generate(prompt, steps)
        result["batch_single_gpu"] = Qwen3Runner(full, batch=len(prompts)).generate_batch(prompts, steps)[0]
        logits_single = prompt_logits(full, None)
        diff = logits_tp.astype(np.float64) - logits_single
        result.update(tokens_single=tokens_single,
                      logit_rel_l2=float(np.sqrt((diff ** 2).sum() / (logits_single.astype(np.float64) ** 2).sum())),
                      logit_cosine=float((logits_tp.astype(np.float64) * logits_single).sum()
                                         / np.linalg.norm(logits_tp.astype(np.float64)) / np.linalg.norm(logits_single.astype(np.float64))),
                      argmax_equal=bool(logits_tp.argmax() == logits_single.argmax()),
                      device_status=list(ops.device_status()))
    gathered = [None] * tp
    dist.all_gather_object(gathered, result)
    if rank == 0:
        print("RESULT " + json.dumps(gathered), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)  # captured graphs hold NCCL work: skip the communicator teardown


if __name__ == "__main__":
    main()
