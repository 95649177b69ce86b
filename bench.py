#!/usr/bin/env python
"""Benchmark of the W8A8 linear-layer hot path on B200.

Workload (N=1): the Qwen3-8B decode GEMM set -- M in {1,4,16} tokens times the five projections
QKV 4096->6144, O 4096->4096, gate_up 4096->24576, down 12288->4096, lm_head 4096->151936 --
each as `quantize` (bf16 activations -> int8 + per-token scale) followed by `linear`
(int8 x int8 -> int32, dequantizing epilogue -> bf16).  One step = one pass over all 15.
Seeded synthetic tensors: activations bf16 N(0,1) with 8 outlier channels x20, weights fp32
N(0,0.02) quantized per output channel.  Metric: algorithmic HBM bytes per second.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N>1 runs under torchrun: tensor-parallel shards (QKV/gate_up/lm_head split by output channel,
O/down split along K with a bf16 NCCL all-reduce of the [M,4096] outputs).
`--impl reference` times the CPU restatement of the reference's CPU-integer path (oracle/) on
the host cores.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SHAPES = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 24576), ("down", 12288, 4096),
          ("lm_head", 4096, 151936)]
DECODE_M = [1, 4, 16]
PREFILL_M = [129, 512, 4096]
ROW_SPLIT = {"o", "down"}  # sharded along K under tensor parallelism, all-reduce after
METRIC = "W8A8 decode GEMM set (Qwen3-8B shapes, M in {1,4,16}): algorithmic HBM GB/s"
WORKLOAD = "configs[1]: quantize+linear over 5 Qwen3-8B projections x M in {1,4,16}"

# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes, per kernel family, from the ncu captures
# summarised under profiles/ (captured on the 50 MB and 100 MB projections; traffic grows with the weight bytes, so
# the ratio is applied to the bench's average algorithmic bytes per launch).
NCU_TRAFFIC_RATIO = {"gemv_mma": 1.025, "gemv_dp4a": 1.035, "gemm_skinny": 1.003}


def kernel_family(M, weight_bytes, K, forced=0):
    """Which kernel w8a8_linear picks (mirrors pick_variant in inferrous_b200/csrc/capi.cu)."""
    names = {1: "naive_linear", 2: "gemv_dp4a", 3: "gemv_mma", 4: "gemm_tcgen05", 5: "gemm_skinny", 8: "gemm_tcgen05_pair", 9: "gemm_cluster"}
    if forced:
        return names[forced]
    if M <= 1:
        return "gemv_dp4a"
    if M <= 8:
        return "gemv_mma"
    if M <= 16:
        return "gemm_skinny" if weight_bytes >= (256 << 20) else "gemv_mma"
    if M <= 64:
        return "gemm_skinny" if weight_bytes >= (64 << 20) else "gemm_cluster"
    if M <= 128:
        if weight_bytes >= (256 << 20):
            return "gemm_skinny"
        return "gemm_cluster" if K >= 8192 and weight_bytes < (64 << 20) else "gemm_tcgen05"
    if M <= 256 and K >= 8192 and weight_bytes < (64 << 20):
        return "gemm_cluster"
    return "gemm_tcgen05_pair"


def linear_bytes(M, K, N):
    return N * K + 4 * N + M * K + 4 * M + 2 * M * N


def quant_bytes(M, K):
    return 2 * M * K + M * K + 4 * M


def shard(name, K, N, tp):
    from inferrous_b200.tp import shard_shape
    return shard_shape(name, K, N, tp)


def workload_config(tp):
    """The `config` object of the JSON line: the workload only, identical for both arms (`--impl ours` / `reference`).
    How an arm executes it (launch mode, collective) is reported under `execution`."""
    per_rank = sum(shard(n, K, N, tp)[0] * shard(n, K, N, tp)[1] for n, K, N in SHAPES)
    step_bytes = sum(linear_bytes(M, *shard(n, K, N, tp)) + quant_bytes(M, shard(n, K, N, tp)[0]) for M in DECODE_M for n, K, N in SHAPES)
    l2_bytes = 126 << 20
    if per_rank >= 2 * l2_bytes:
        l2 = (f"weights ({per_rank >> 20} MiB streamed per pass and rank, each matrix revisited only after all the others) "
              "exceed the 126 MB L2; no flush")
    else:
        l2 = (f"weights per rank ({per_rank >> 20} MiB per pass) do not exceed twice the 126 MB L2: the pass rotates over "
              f"{weight_copies(tp)} copies of every matrix, so that more than twice the L2 is streamed between two visits of a copy; no flush")
    return {"workload": WORKLOAD, "shapes": {n: [K, N] for n, K, N in SHAPES}, "M": DECODE_M,
            "parallelism": f"tp{tp}" if tp > 1 else "single", "l2": l2, "bytes_per_step": step_bytes}


def weight_copies(tp):
    """Distinct copies of every weight matrix that a rank rotates over, so that its passes stream from HBM, not from L2."""
    per_rank = sum(shard(n, K, N, tp)[0] * shard(n, K, N, tp)[1] for n, K, N in SHAPES)
    return max(1, -(-2 * (126 << 20) // per_rank))


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            try:
                import torch
                pr = torch.cuda.get_device_properties(index)
                bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
                self.h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _sample(self):
        nv = self.nv
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                     "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                     "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
            for k, bit in names.items():
                if r & bit:
                    self.reasons.add(k)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._sample()
            time.sleep(0.005)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread:
            self._sample()
            self._stop.set()
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_weights_device(torch, K, N, seed):
    """fp32 N(0,0.02) -> per-output-channel symmetric int8 (tools/prepare.py:79-81), generated on the device."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.empty((N, K), dtype=torch.int8, device="cuda")
    s = torch.empty((N,), dtype=torch.float32, device="cuda")
    rows = max(1, (64 << 20) // K)
    for r0 in range(0, N, rows):
        w = torch.randn((min(rows, N - r0), K), generator=g, device="cuda", dtype=torch.float32) * 0.02
        sc = w.abs().amax(1, keepdim=True).clamp(min=1e-8) / 127.0
        q[r0:r0 + w.shape[0]] = torch.round(w / sc).clamp(-127, 127).to(torch.int8)
        s[r0:r0 + w.shape[0]] = sc.flatten()
    return q, s


def make_activations_device(torch, M, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((M, K), generator=g, device="cuda", dtype=torch.float32)
    cols = torch.randperm(K, generator=g, device="cuda")[:8]
    x[:, cols] *= 20.0
    return x.to(torch.bfloat16)


def run_ours(args):
    import torch
    import torch.distributed as dist

    from inferrous_b200 import ops
    from inferrous_b200.tp import all_reduce_sum

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    tp = world
    torch.cuda.set_device(local)
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"  # NCCL would print its version on stdout, which carries the one JSON line
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ops.init(local)
    ops.set_programmatic_launch(not args.no_pdl)
    # Sum of the row-split partial outputs: NCCL, or (--peer-allreduce) the library's one-shot peer-memory kernel.
    reducer, reduce_kind, reduce_check = None, "none", None
    fused = None  # row-split projections with the all-reduce fused in (w8a8_linear_allreduce)
    if world > 1:
        reduce_kind = "nccl"
        if args.fused_allreduce and not args.peer_allreduce and world <= args.fused_max_ranks:
            try:
                from inferrous_b200.tp import PeerLinear
                fused = PeerLinear(dist.group.WORLD, max(DECODE_M) * 4096)
                # self-check before anything is timed: fused result == projection, all-gather, sum in rank order (bit for bit)
                gen = torch.Generator(device="cuda").manual_seed(1000 + rank)
                cw = torch.randint(-127, 128, (4096, 512), dtype=torch.int8, device="cuda", generator=gen)
                cmat = ops.Matrix(cw, torch.full((4096,), 1e-4, dtype=torch.float32, device="cuda"))
                agree = torch.ones(1, device="cuda")
                for rows in (1, 4, 16, 1):
                    cq = torch.randint(-127, 128, (rows, 512), dtype=torch.int8, device="cuda", generator=gen)
                    cs = torch.full((rows,), 0.01, dtype=torch.float32, device="cuda")
                    got = torch.empty(rows, 4096, dtype=torch.bfloat16, device="cuda")
                    fused.linear_residual(cq, cs, cmat, got, None, None)
                    part = torch.empty_like(got)
                    ops.linear_quantized(cq, cs, cmat, part)
                    parts = [torch.empty_like(part) for _ in range(world)]
                    dist.all_gather(parts, part)
                    total = torch.zeros(rows, 4096, dtype=torch.float32, device="cuda")
                    for p in parts:
                        total = total + p.float()
                    if not torch.equal(got, total.to(torch.bfloat16)):
                        agree.zero_()
                dist.all_reduce(agree, op=dist.ReduceOp.MIN)
                if agree.item() < 1.0 or ops.device_status()[0] != 0:
                    raise RuntimeError("fused result differs from the sum of the gathered partial outputs")
                del cmat, cw
                reduce_kind = "fused_into_projection_over_peer_memory"
                reduce_check = "bit-identical to projection + all-gather + sum in rank order (4 seeded calls)"
            except Exception as exc:
                print(f"bench: fused projection + all-reduce unavailable ({exc}); using NCCL", file=sys.stderr)
                fused = None
        elif args.peer_allreduce:
            try:
                from inferrous_b200.tp import PeerAllReduce
                reducer = PeerAllReduce(dist.group.WORLD, slot_elems=max(DECODE_M) * 4096)
                # self-check against NCCL on seeded data before anything is timed
                t = (torch.randn(16 * 4096, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rank)) * 3).to(torch.bfloat16)
                ref = t.float().clone()
                dist.all_reduce(ref)
                got = reducer.all_reduce(t.clone())
                torch.cuda.synchronize()
                err = (got.float() - ref).abs().max().item() / max(1e-6, ref.abs().max().item())
                same = torch.tensor([1.0 if err < 2e-2 else 0.0], device="cuda")
                dist.all_reduce(same, op=dist.ReduceOp.MIN)
                if same.item() < 1.0:
                    raise RuntimeError(f"peer all-reduce differs from NCCL (rel err {err:.3g})")
                reduce_kind, reduce_check = "peer_memory_one_shot", f"max rel err vs f32 NCCL sum {err:.2e}"
            except Exception as exc:
                print(f"bench: peer-memory all-reduce unavailable ({exc}); using NCCL", file=sys.stderr)
                reducer = None
    hbm_peak, _, peak_kind = measured_peaks()

    # ---- resident weights (model state) and per-(M,shape) activation/output buffers ----
    # A rank whose shard of the weights is smaller than twice the L2 rotates over several distinct copies of every matrix
    # (one copy per step, round-robin), so that its passes stream from HBM instead of from the cache.
    copies = weight_copies(tp)
    mats_all, bufs = [], {}
    for c in range(copies):
        mats_c = {}
        for i, (name, K, N) in enumerate(SHAPES):
            k, n = shard(name, K, N, tp)
            wq, ws = make_weights_device(torch, k, n, seed=1000 + 10 * i + rank + 100 * c)
            mats_c[name] = ops.Matrix(wq, ws)
        mats_all.append(mats_c)
    mats = mats_all[0]
    # Activations and outputs of one step live in two device arenas mirrored by two pinned host arenas, so the
    # end-to-end step moves them with one host->device and one device->host copy.
    def carve(sizes):
        offs, total = [], 0
        for n_el in sizes:
            offs.append(total)
            total += (n_el + 127) // 128 * 128  # 256-byte aligned bf16 slices
        return offs, total
    keys = [(M, name, *shard(name, K, N, tp)) for M in DECODE_M for name, K, N in SHAPES]
    x_off, x_tot = carve([M * k for M, _, k, _ in keys])
    y_off, y_tot = carve([M * n for M, _, _, n in keys])
    x_all = torch.empty(x_tot, dtype=torch.bfloat16, device="cuda")
    y_all = torch.empty(y_tot, dtype=torch.bfloat16, device="cuda")
    hx_all = torch.empty(x_tot, dtype=torch.bfloat16).pin_memory()
    hy_all = torch.empty(y_tot, dtype=torch.bfloat16).pin_memory()
    for i, (M, name, k, n) in enumerate(keys):
        x = x_all[x_off[i]:x_off[i] + M * k].view(M, k)
        x.copy_(make_activations_device(torch, M, k, seed=7 * M + i + 100 * rank))
        bufs[(M, name)] = dict(
            x=x,
            q=torch.empty((M, k), dtype=torch.int8, device="cuda"),
            s=torch.empty((M,), dtype=torch.float32, device="cuda"),
            y=y_all[y_off[i]:y_off[i] + M * n].view(M, n))
    hx_all.copy_(x_all)
    torch.cuda.synchronize()

    step_bytes = 0
    for M in DECODE_M:
        for name, K, N in SHAPES:
            k, n = shard(name, K, N, tp)
            step_bytes += linear_bytes(M, k, n) + quant_bytes(M, k)
    total_bytes = step_bytes * world  # every rank moves the same amount

    gemv_events = []  # (kernel family, bytes, start, end) per linear launch of the timed region

    def step(record=False, host_io=False, ms=None, copy=0):
        mats = mats_all[copy]
        if host_io:
            x_all.copy_(hx_all, non_blocking=True)
        for M in (DECODE_M if ms is None else ms):
            for name, K, N in SHAPES:
                b = bufs[(M, name)]
                k, n = shard(name, K, N, tp)
                ops.quantize(b["x"], b["q"], b["s"])
                if record:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                if fused is not None and name in ROW_SPLIT and not record:
                    fused.linear_residual(b["q"], b["s"], mats[name], b["y"], None, None)  # GEMV that pushes + consumer
                    continue
                ops.linear_quantized(b["q"], b["s"], mats[name], b["y"], args.variant)
                if record:
                    e1.record()
                    gemv_events.append((kernel_family(M, k * n, k, args.variant), linear_bytes(M, k, n), e0, e1))
                if world > 1 and name in ROW_SPLIT:
                    if reducer is not None:
                        reducer.all_reduce(b["y"])  # one kernel: push to peers, wait, sum in rank order
                    else:
                        all_reduce_sum(b["y"])  # bf16 NCCL all-reduce of the partial outputs [M,4096]

    # End to end, one step: inputs up, every projection, outputs down.  The outputs of a token count form one contiguous
    # span of the arena; the largest count runs first, so that its span (three quarters of the bytes) travels to the host
    # on a second stream while the smaller counts compute, and only the smallest span is left uncovered at the end.
    y_span = {}
    for i, (M, _, _, n) in enumerate(keys):
        lo, hi = y_span.get(M, (y_off[i], y_off[i]))
        y_span[M] = (lo, y_off[i] + (M * n + 127) // 128 * 128)
    copy_stream = torch.cuda.Stream()

    def step_e2e(copy=0):
        main = torch.cuda.current_stream()
        x_all.copy_(hx_all, non_blocking=True)
        for M in sorted(DECODE_M, reverse=True):
            step(ms=[M], copy=copy)
            lo, hi = y_span[M]
            ready = torch.cuda.Event()
            ready.record(main)
            copy_stream.wait_event(ready)
            with torch.cuda.stream(copy_stream):
                hy_all[lo:hi].copy_(y_all[lo:hi], non_blocking=True)
        main.wait_stream(copy_stream)

    def timed(fn, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([t0.elapsed_time(t1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.barrier()
        return float(ms.item())

    def capture_one(fn):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            fn()
        return g

    class Rotation:
        """One step per call, over the weight copies in turn (copy = call number mod copies)."""

        def __init__(self, fns):
            self.fns, self.turn = fns, 0

        def __call__(self):
            self.fns[self.turn % len(self.fns)]()
            self.turn += 1

    def capture(fn):
        """One step as a CUDA graph per weight copy (the reference replays captured decode graphs, src/gpu.rs:318-328,890).
        Every launch call of the library is capture-safe; under TP the NCCL all-reduce is captured with it."""
        graphs = [capture_one(lambda c=c: fn(copy=c)) for c in range(copies)]
        return graphs, Rotation([g.replay for g in graphs])

    if fused is not None:
        # One eager step first: if a wait for another rank's packets ran out (the kernels give up after two seconds and
        # report it), every rank falls back to NCCL together rather than timing a broken exchange.
        step()
        expired = torch.tensor([float(ops.device_status()[0] != 0)], device="cuda")
        dist.all_reduce(expired, op=dist.ReduceOp.MAX)
        if expired.item() > 0:
            print("bench: a wait in the fused projection + all-reduce expired; using NCCL", file=sys.stderr)
            fused, reduce_kind = None, "nccl"
    for _ in range(max(args.warmup, copies)):
        step()
    launch_mode = "eager"
    run_step = Rotation([lambda c=c: step(copy=c) for c in range(copies)])
    graph = e2e_graph = None
    if not args.eager:
        try:
            graph, run_step = capture(step)
            launch_mode = "cuda_graph"
            for _ in range(args.warmup):
                run_step()
        except Exception as exc:  # keep measuring, say why
            print(f"bench: CUDA graph capture failed ({exc}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    ms = timed(run_step, args.steps)
    clocks = sampler.stop()
    ms_per_step = ms / args.steps
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # per-launch CUDA events need eager launches: the same steps again, instrumented
    eager_ms = timed(Rotation([lambda c=c: step(record=True, copy=c) for c in range(copies)]), args.steps) / args.steps

    # ---- roofline of the dominant kernel family ----
    # Per-launch events (above) bracket one short kernel each and carry several microseconds of event and launch
    # latency per launch.  Where a family's launches stream more weight bytes than twice the L2, the family is timed
    # again as a batch: its linear launches of one step back to back, K steps between ONE pair of events, so that the
    # latency is paid once per K steps and every matrix is still revisited only after the others displaced it.
    fam = {}
    for name, nbytes, e0, e1 in gemv_events:
        d = fam.setdefault(name, [0, 0.0, 0])
        d[0] += nbytes
        d[1] += e0.elapsed_time(e1) * 1e-3
        d[2] += 1
    members = {}
    for M in DECODE_M:
        for name, K, N in SHAPES:
            k, n = shard(name, K, N, tp)
            members.setdefault(kernel_family(M, k * n, k, args.variant), []).append((M, name, linear_bytes(M, k, n), k * n))
    batched = {}
    for family, items in members.items():
        if sum({name: wbytes for _, name, _, wbytes in items}.values()) < 2 * (126 << 20):
            continue

        def run_family(items=items):
            for M, name, _, _ in items:
                b = bufs[(M, name)]
                ops.linear_quantized(b["q"], b["s"], mats[name], b["y"], args.variant)

        for _ in range(3):
            run_family()
        family_ms = timed(run_family, args.steps)
        batched[family] = [sum(i[2] for i in items) * args.steps, family_ms * 1e-3, len(items) * args.steps]
    per_launch = {k: {"achieved": round(v[0] / v[1] / 1e9, 1), "avg_launch_us": round(v[1] / v[2] * 1e6, 2)} for k, v in fam.items()}
    fam.update(batched)
    dominant = max(fam, key=lambda k: fam[k][1])
    dom_bytes, dom_s, dom_n = fam[dominant]
    achieved = dom_bytes / dom_s / 1e9
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": round(achieved, 1), "peak": hbm_peak, "peak_kind": peak_kind,
                "unit": "GB/s", "frac": round(achieved / hbm_peak, 4),
                "traffic": int(dom_bytes / dom_n * NCU_TRAFFIC_RATIO[dominant]) if dominant in NCU_TRAFFIC_RATIO else None,
                "algorithmic_bytes_per_launch": dom_bytes // dom_n, "avg_launch_us": round(dom_s / dom_n * 1e6, 2),
                "launches": dom_n,
                "timing": ("CUDA events around the family's linear launches of K steps, launched eagerly back to back right after "
                           "the timed region" if dominant in batched else
                           "per-launch CUDA events over the same K steps launched eagerly right after the timed region")
                          + f" ({eager_ms:.4f} ms/step eager with per-launch events)",
                "per_launch_events": per_launch,
                "other_kernels": {k: {"achieved": round(v[0] / v[1] / 1e9, 1), "frac": round(v[0] / v[1] / 1e9 / hbm_peak, 4),
                                      "launches": v[2]} for k, v in fam.items() if k != dominant}}

    # ---- end to end: host buffers in, host buffers out, through the same calls ----
    e2e_step = Rotation([lambda c=c: step_e2e(copy=c) for c in range(copies)])
    for _ in range(3):
        e2e_step()
    if launch_mode == "cuda_graph":
        try:
            e2e_graph, e2e_step = capture(step_e2e)
            for _ in range(3):
                e2e_step()
        except Exception as exc:
            print(f"bench: e2e graph capture failed ({exc}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
    e2e_ms = timed(e2e_step, args.steps) / args.steps
    h2d = x_all.numel() * 2
    d2h = y_all.numel() * 2
    e2e = {"value": round(total_bytes / (e2e_ms * 1e-3) / 1e9, 1), "unit": "GB/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 4),
           "note": "activations from pinned host memory and outputs back to it every step, the copy of each token count's outputs "
                   "overlapped with the projections of the next; weights resident (model state)"}

    extra = {}
    if world == 1 and not args.no_extra:
        extra["per_shape"] = per_shape_table(torch, ops, mats, bufs, hbm_peak, args.variant)
        extra["prefill"] = prefill_table(torch, ops, mats, args.prefill_variant)
        extra["roofline_prefill"] = prefill_roofline(extra["prefill"], hbm_peak)
        if not args.shapes:
            extra["quantizers"] = quantizer_table(torch, ops, hbm_peak)
            extra["decode_fused_kernels"] = decode_fused_table(torch, ops, hbm_peak)
        body = sum(r["us"] for r in extra["per_shape"] if r["M"] == 1 and r["shape"] != "lm_head")
        head = sum(r["us"] for r in extra["per_shape"] if r["M"] == 1 and r["shape"] == "lm_head")
        if body > 0 and head > 0:
            extra["decode_linear_only_tok_s_estimate"] = round(1e6 / (36 * body + head), 1)
    if not args.no_extra and not args.shapes and not args.no_model:
        # A shape the library rejects raises before any kernel or collective is queued, identically on every rank, so
        # reporting the error instead of the table cannot leave ranks waiting for one another.
        try:
            extra["qwen3_8b_generation"] = model_generation_table(torch, hbm_peak, rank, world, dist.group.WORLD if world > 1 else None,
                                                                  fused_allreduce=fused is not None)
        except (ValueError, RuntimeError) as exc:
            extra["qwen3_8b_generation"] = {"error": f"{type(exc).__name__}: {exc}"}

    # quantize + linear per projection, plus the packet consumer of every fused projection + all-reduce
    launches_per_step = (2 * len(SHAPES) + (sum(1 for n, _, _ in SHAPES if n in ROW_SPLIT) if fused is not None else 0)) * len(DECODE_M)
    out = {"metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
           "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "int8xint8->int32 (bf16 in/out)",
           "data": "synthetic", "impl": "ours",
           "config": workload_config(world),
           "execution": {"launch": launch_mode + ("" if args.no_pdl else "+programmatic_dependent_launch"),
                         "all_reduce": reduce_kind, "all_reduce_check": reduce_check, "weight_copies": copies},
           "roofline": roofline, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks}
    if world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(torch, mats, bufs, reps=3)
    out.update(extra)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        # Captured graphs hold NCCL work of this process group: release them before the group, and do not let
        # a slow communicator teardown keep the job alive after the result is out.
        graph = e2e_graph = run_step = e2e_step = None
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def time_launch(torch, fn, iters, flush):
    """Median device time of fn() with the L2 displaced before every timed launch.  The displacement is a READ of a
    buffer twice the size of L2: it leaves clean lines behind, so the timed kernel does not pay for writing back
    somebody else's dirty data."""
    ts = []
    for _ in range(iters):
        flush.sum()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts)


def per_shape_table(torch, ops, mats, bufs, hbm_peak, variant=0):
    flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")
    rows = []
    for M in DECODE_M:
        for name, K, N in SHAPES:
            b = bufs[(M, name)]
            us = time_launch(torch, lambda: ops.linear_quantized(b["q"], b["s"], mats[name], b["y"], variant), 20, flush)
            gbs = linear_bytes(M, K, N) / us / 1e3
            rows.append({"shape": name, "M": M, "us": round(us, 2), "GB/s": round(gbs, 1), "frac_hbm": round(gbs / hbm_peak, 3)})
    # the allocation-free entry point (raw weight pointers, scratch in a fixed device array) on the O projection
    if 16 in DECODE_M and "o" in mats:
        b, m = bufs[(16, "o")], mats["o"]
        us = time_launch(torch, lambda: ops.linear_no_alloc(b["q"], b["s"], m.w, m.scale, b["y"]), 20, flush)
        gbs = linear_bytes(16, m.k, m.n) / us / 1e3
        rows.append({"shape": "o via w8a8_linear_no_alloc", "M": 16, "us": round(us, 2), "GB/s": round(gbs, 1),
                     "frac_hbm": round(gbs / hbm_peak, 3)})
    del flush
    return rows


def prefill_table(torch, ops, mats, variant=0):
    """Tensor-core regime, reported beside the headline: quantize + GEMM at M in {129,512,4096}."""
    flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")
    rows = []
    for M in PREFILL_M:
        for name, K, N in SHAPES:
            x = make_activations_device(torch, M, K, seed=M)
            q = torch.empty((M, K), dtype=torch.int8, device="cuda")
            s = torch.empty((M,), dtype=torch.float32, device="cuda")
            y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
            ops.quantize(x, q, s)
            ops.linear_quantized(q, s, mats[name], y, variant)
            us = time_launch(torch, lambda: ops.linear_quantized(q, s, mats[name], y, variant), 5, flush)
            rows.append({"shape": name, "M": M, "us": round(us, 1), "TOPS": round(2.0 * M * N * K / us / 1e6, 1),
                         "GB/s": round(linear_bytes(M, K, N) / us / 1e3, 1)})
            del x, q, s, y
    del flush
    return rows


INT8_NOMINAL_TOPS = 4500.0  # dense INT8 tensor peak of a B200 (no measured INT8 figure is available)


def prefill_roofline(rows, hbm_peak):
    """The tensor-core regime beside the headline's HBM roofline: per (M, projection) the time against
    max(ops / INT8 peak, algorithmic bytes / HBM peak), and which of the two terms binds.  At 129 rows every
    projection is bound by the one pass over its weights (about 240 ops per byte against a ridge of 560 or more); from
    512 rows up by the tensor cores.  Peaks: 4500 TOPS nominal dense INT8, and for comparison twice the measured bf16
    cuBLAS burst; the HBM peak is the measured copy rate."""
    _, bf16_tflops, kind = measured_peaks()
    shapes = {n: (K, N) for n, K, N in SHAPES}
    per_shape, best = [], None
    for r in rows:
        K, N = shapes[r["shape"]]
        M, us = r["M"], r["us"]
        ops_total = 2.0 * M * N * K
        t_tensor = ops_total / (INT8_NOMINAL_TOPS * 1e12) * 1e6
        t_hbm = linear_bytes(M, K, N) / (hbm_peak * 1e9) * 1e6
        bound = "tensor" if t_tensor >= t_hbm else "hbm"
        row = {"shape": r["shape"], "M": M, "us": us, "TOPS": r["TOPS"], "GB/s": r["GB/s"], "bound": bound,
               "floor_us": round(max(t_tensor, t_hbm), 2), "frac": round(max(t_tensor, t_hbm) / us, 3),
               "frac_of_2x_measured_bf16": round(r["TOPS"] / (2 * bf16_tflops), 3) if bf16_tflops else None}
        per_shape.append(row)
        if bound == "tensor" and (best is None or ops_total > best[0]):
            best = (ops_total, row)
    top = best[1] if best else None
    return {"bound": "tensor", "kernel": "gemm_tcgen05_pair (tcgen05.mma.cta_group::2.kind::i8)",
            "achieved": top and top["TOPS"], "peak": INT8_NOMINAL_TOPS, "peak_kind": "nominal dense INT8", "unit": "TOPS",
            "frac": top and round(top["TOPS"] / INT8_NOMINAL_TOPS, 4), "shape": top and f'{top["shape"]} at M={top["M"]}',
            "twice_measured_bf16_tflops": round(2 * bf16_tflops, 1), "bf16_peak_kind": kind,
            "timing": "median of 5 launches, CUDA events, L2 displaced by a 256 MB read before every launch",
            "per_shape": per_shape}


def quantizer_table(torch, ops, hbm_peak):
    """The activation quantizers of configs[2]: fused with RMSNorm (QKV / gate_up input, K=4096) and with SwiGLU
    (down input, [M,24576] -> [M,12288]); HBM-bound.  Bytes: 2MK in + MK out + 4M (+2K gamma); SwiGLU reads 4MI.
    Timed as 8 back-to-back launches over rotating buffer sets that together exceed the L2 (single launches of a
    few microseconds are below what a CUDA-event pair resolves), replayed as one CUDA graph."""
    rows = []
    K, I = 4096, 12288
    for M in DECODE_M + PREFILL_M:
        sets = max(2, min(8, (300 << 20) // max(1, 5 * M * I)))  # enough copies to push the working set past the L2
        xs = [make_activations_device(torch, M, K, seed=M + i) for i in range(sets)]
        gus = [make_activations_device(torch, M, 2 * I, seed=M + 50 + i) for i in range(sets)]
        gamma = (1.0 + 0.1 * torch.randn(K, device="cuda")).to(torch.bfloat16)
        q4 = [torch.empty((M, K), dtype=torch.int8, device="cuda") for _ in range(sets)]
        q12 = [torch.empty((M, I), dtype=torch.int8, device="cuda") for _ in range(sets)]
        s = torch.empty((M,), dtype=torch.float32, device="cuda")
        cases = [("quantize", lambda i: ops.quantize(xs[i], q4[i], s), 3 * M * K + 4 * M),
                 ("rmsnorm_quantize", lambda i: ops.norm_quantize(xs[i], gamma, None, q4[i], s, None), 3 * M * K + 4 * M + 2 * K),
                 ("swiglu_quantize", lambda i: ops.swiglu_quantize(gus[i][:, :I], gus[i][:, I:], q12[i], s), 5 * M * I + 4 * M)]
        for name, fn, nbytes in cases:
            reps = 8
            for i in range(sets):
                fn(i)
            torch.cuda.synchronize()
            # the eight launches are replayed as one CUDA graph, so that what is timed is the kernels, not the cost of
            # eight host calls (a few microseconds each, more than a quantizer launch of a few rows takes)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for r in range(reps):
                    fn(r % sets)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            e1.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            del graph
            rows.append({"kernel": name, "M": M, "us": round(us, 2), "GB/s": round(nbytes / us / 1e3, 1),
                         "frac_hbm": round(nbytes / us / 1e3 / hbm_peak, 3), "buffer_sets": sets})
        del xs, gus, q4, q12
    return rows


def decode_fused_table(torch, ops, hbm_peak):
    """The fused decode kernels the reference publishes per-kernel numbers for (docs/qwen3-8b-w8a8/optimization/
    round-6.md:11-13, on an RTX PRO 6000): gate+up+SwiGLU, O and down with residual, grouped Q/K/V; 1 token."""
    flush = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")
    mk = lambda K, N, seed: ops.Matrix(*make_weights_device(torch, K, N, seed))
    act = lambda n: torch.empty((1, n), dtype=torch.bfloat16, device="cuda")
    q4 = torch.randint(-127, 128, (1, 4096), dtype=torch.int8, device="cuda")
    q12 = torch.randint(-127, 128, (1, 12288), dtype=torch.int8, device="cuda")
    s = torch.full((1,), 0.01, dtype=torch.float32, device="cuda")
    wg, wu, wo, wd = mk(4096, 12288, 1), mk(4096, 12288, 2), mk(4096, 4096, 3), mk(12288, 4096, 4)
    wq, wk, wv = mk(4096, 4096, 5), mk(4096, 1024, 6), mk(4096, 1024, 7)
    g, u, a = act(12288), act(12288), act(12288)
    mx = torch.zeros(1, dtype=torch.int32, device="cuda")
    res, y, comb = act(4096), act(4096), act(4096)
    oq, ok_, ov = act(4096), act(1024), act(1024)
    cases = [("linear_swiglu (gate+up, 100.7 MB)", lambda: ops.linear_swiglu(q4, s, wg, wu, g, u, a, mx), 2 * 12288 * 4096, 63.22),
             ("linear_residual O (16.8 MB)", lambda: ops.linear_residual(q4, s, wo, y, res, comb), 4096 * 4096, 11.94),
             ("linear_residual down (50.3 MB)", lambda: ops.linear_residual(q12, s, wd, y, res, comb), 4096 * 12288, 33.94),
             ("linear_triple QKV (25.2 MB)", lambda: ops.linear_grouped(q4, s, [wq, wk, wv], [oq, ok_, ov]), 6144 * 4096, 16.91)]
    # the reference's own output head (bf16 weights, its summation order) with the greedy selection fused in, and the
    # W8A8 head that BASELINE.json names: one row against [151936, 4096]
    vocab = 151936
    head_w = torch.empty((vocab, 4096), dtype=torch.bfloat16, device="cuda").normal_(0.0, 0.02)
    head_x = torch.randn((1, 4096), device="cuda").to(torch.bfloat16)
    token = torch.zeros(1, dtype=torch.int32, device="cuda")
    cases.append(("head, bf16 weights (1245 MB) + select_token", lambda: ops.head_bf16(head_x, head_w, token=token), 2 * vocab * 4096, None))
    wh = mk(4096, vocab, 8)
    cases.append(("head, W8A8 (622 MB) + select_token", lambda: ops.linear_argmax(q4, s, wh, token), vocab * 4096, None))
    rows = []
    for name, fn, wbytes, ref_us in cases:
        fn()
        us = time_launch(torch, fn, 20, flush)
        rows.append({"kernel": name, "us": round(us, 2), "GB/s": round(wbytes / us / 1e3, 1),
                     "frac_hbm": round(wbytes / us / 1e3 / hbm_peak, 3), "reference_us_rtx_pro_6000": ref_us})
    return rows


def model_generation_table(torch, hbm_peak, rank=0, world=1, group=None, fused_allreduce=True):
    """Whole-model greedy generation of the Qwen3-8B architecture with random-init weights (inferrous_b200.qwen3):
    the prompt / generated lengths the reference's decode table uses (docs/qwen3-8b-w8a8/benchmarks.md:13-15: prompt
    5 / 129 / 512, 32 generated) plus the 129 + 128 run.  Host-visible time per step: control upload, graph replay,
    token read-back, as the reference's generate() measures it (src/gpu.rs:873-908).  With several GPUs the model is
    tensor-parallel (heads, gate/up channels and vocabulary split; bf16 all-reduce after O and down), every rank
    generates in lockstep and the slowest rank's time counts."""
    import numpy as np
    import torch.distributed as dist

    from inferrous_b200.qwen3 import Qwen3Config, Qwen3Runner, Qwen3Weights

    config = Qwen3Config.qwen3_8b()
    full = Qwen3Weights.random(config, seed=0)
    weights = full.shard(rank, world)
    del full
    torch.cuda.empty_cache()
    runner = Qwen3Runner(weights, group=group, fused_allreduce=fused_allreduce)
    exchange = "single GPU"
    if world > 1 and not fused_allreduce:
        exchange = "NCCL all-reduce"
    elif world > 1:
        # two tokens first: if a wait for another rank's packets expired, all ranks switch to NCCL together
        exchange = "fused into the O / down projections over peer memory"
        runner.generate([1, 2, 3], 2, use_graph=False)
        from inferrous_b200 import ops as _ops
        expired = torch.tensor([float(_ops.device_status()[0] != 0)], device="cuda")
        dist.all_reduce(expired, op=dist.ReduceOp.MAX, group=group)
        if expired.item() > 0:
            exchange = "NCCL all-reduce (a wait of the fused exchange expired)"
            runner = Qwen3Runner(weights, group=group, fused_allreduce=False)
    rng = np.random.default_rng(0)
    rows = []
    published = {5: 182.3, 129: 178.2, 512: 170.5}
    for prompt_len, generated in [(5, 32), (129, 32), (512, 32), (129, 128)]:
        prompt = [int(t) for t in rng.integers(0, config.vocab, prompt_len)]
        runner.generate(prompt, generated)  # warm-up: captures the decode graph on first use
        _, seconds = runner.generate(prompt, generated)
        if world > 1:
            slowest = torch.tensor(seconds, dtype=torch.float64, device="cuda")
            dist.all_reduce(slowest, op=dist.ReduceOp.MAX, group=group)
            seconds = slowest.tolist()
        decode = seconds[1:]
        median = float(np.median(decode))
        rows.append({"prompt": prompt_len, "generated": generated, "prefill_ms": round(seconds[0] * 1e3, 3),
                     "decode_ms_per_token_median": round(median * 1e3, 4),
                     "decode_tok_s": round(len(decode) / sum(decode), 1),
                     "weight_GB/s": round(config.weight_bytes() / median / 1e9, 1),
                     "frac_hbm": round(config.weight_bytes() / median / 1e9 / (hbm_peak * world), 3),
                     "reference_tok_s_rtx_pro_6000": published.get(prompt_len) if generated == 32 else None})
    resident = getattr(runner, "plan", None) is not None
    del runner
    torch.cuda.empty_cache()
    table = {"model": "Qwen3-8B architecture, random-init W8A8 weights (body and head int8), batch 1, greedy",
             "parallelism": f"tp{world}" if world > 1 else "single", "all_reduce": exchange,
             "decode_step": (("one resident cooperative kernel for all layers (qwen3_decode_layers) + head"
                              + (", the O / down partial outputs exchanged as packets over peer memory inside it" if world > 1 else ""))
                             if resident
                             else "one launch per operator, CUDA graph with programmatic edges"),
             "weight_bytes_per_token": config.weight_bytes(), "runs": rows}
    if resident:  # the same step as one launch per operator, for comparison
        other = Qwen3Runner(weights, group=group, fused_allreduce=fused_allreduce and not exchange.startswith("NCCL"), resident=False)
        prompt = [int(t) for t in np.random.default_rng(0).integers(0, config.vocab, 129)]
        other.generate(prompt, 32)
        _, seconds = other.generate(prompt, 32)
        if world > 1:
            slowest = torch.tensor(seconds, dtype=torch.float64, device="cuda")
            dist.all_reduce(slowest, op=dist.ReduceOp.MAX, group=group)
            seconds = slowest.tolist()
        median = float(np.median(seconds[1:]))
        table["separate_launches"] = {"prompt": 129, "generated": 32, "decode_ms_per_token_median": round(median * 1e3, 4),
                                      "decode_tok_s": round(len(seconds[1:]) / sum(seconds[1:]), 1)}
        del other
        torch.cuda.empty_cache()
    try:
        table["config4"] = config4_table(torch, weights, config, hbm_peak, rank, world, group,
                                         fused_allreduce and not exchange.startswith("NCCL"))
    except (ValueError, RuntimeError) as exc:
        table["config4"] = {"error": f"{type(exc).__name__}: {exc}"}
    del weights
    torch.cuda.empty_cache()
    return table


def config4_table(torch, weights, config, hbm_peak, rank, world, group, fused_allreduce, sequences=64, timed_steps=16):
    """BASELINE.json configs[4] on the whole model: (i) ragged decode of 64 concurrent sequences whose context lengths are
    drawn uniformly from [128, 4096] (seeded), every step advancing all of them by one token in one pass of 64 rows;
    (ii) one 4096-token prefill.  Prompts are uniform-random token ids; every sequence is really prefilled into its own
    KV cache first.  Host-visible time per decode step (state upload, graph replay, read-back of the 64 tokens), the
    slowest rank's.  Bytes per decode step: the int8 weights once, plus every visible key and value once."""
    import numpy as np
    import torch.distributed as dist

    from inferrous_b200.qwen3 import Qwen3Runner, Workspace

    full = weights.full_config
    rng = np.random.default_rng(4)
    warm = 3
    total_steps = warm + timed_steps
    contexts = [int(n) for n in rng.integers(128, 4097, sequences)]
    # a sequence must be able to grow by the decode steps that are timed: the longest contexts start that many tokens short
    prompt_lens = [min(n, full.context - total_steps - 1) for n in contexts]
    prompts = [[int(t) for t in rng.integers(0, full.vocab, n)] for n in prompt_lens]
    def run(**kw):
        runner = Qwen3Runner(weights, group=group, batch=sequences, **kw)
        runner.generate_batch(prompts, 2)  # captures the step graph; also the first check of the exchange at 64 rows
        ok = True
        if world > 1 and kw.get("fused_allreduce", True):
            from inferrous_b200 import ops as _ops
            expired = torch.tensor([float(_ops.device_status()[0] != 0)], device="cuda")
            dist.all_reduce(expired, op=dist.ReduceOp.MAX, group=group)
            ok = expired.item() == 0
        toks, secs = runner.generate_batch(prompts, 1 + total_steps)
        if world > 1:
            slowest = torch.tensor(secs, dtype=torch.float64, device="cuda")
            dist.all_reduce(slowest, op=dist.ReduceOp.MAX, group=group)
            secs = slowest.tolist()
        del runner
        torch.cuda.empty_cache()
        return ok, toks, secs

    # Under tensor parallelism the sum after O and down is timed both ways at 64 rows: fused into the projection (tagged
    # packets to every rank) and as projection + NCCL all-reduce + residual kernel; the step reports the faster one.
    exchange_ms = {}
    ok, tokens, seconds = run(fused_allreduce=False) if world > 1 else run()
    exchange = "NCCL all-reduce" if world > 1 else "single GPU"
    if world > 1:
        exchange_ms["nccl"] = round(float(np.median(seconds[1 + warm:])) * 1e3, 4)
        if fused_allreduce:
            ok_f, tokens_f, seconds_f = run(fused_allreduce=True, peer_rows_times_ranks=1 << 30)
            if ok_f:
                exchange_ms["fused_packets"] = round(float(np.median(seconds_f[1 + warm:])) * 1e3, 4)
                if exchange_ms["fused_packets"] < exchange_ms["nccl"]:
                    tokens, seconds, exchange = tokens_f, seconds_f, "fused into the O / down projections over peer memory"
    decode = seconds[1 + warm:]
    median = float(np.median(decode))
    # keys visible to step s of the timed region: prompt + warm + s + 1 per sequence (the new token's own key included)
    mid = warm + timed_steps // 2
    kv_bytes = sum(p + mid + 1 for p in prompt_lens) * full.layers * 2 * full.kv_heads * 128 * 2
    step_bytes = full.weight_bytes() + kv_bytes
    ragged = {"sequences": sequences, "context_min": min(contexts), "context_max": max(contexts),
              "context_mean": round(sum(contexts) / sequences, 1), "prefill_all_sequences_s": round(seconds[0], 3),
              "timed_steps": timed_steps, "decode_ms_per_step_median": round(median * 1e3, 4),
              "tok_s": round(sequences * len(decode) / sum(decode), 1),
              "bytes_per_step": step_bytes, "kv_bytes_per_step": kv_bytes,
              "GB/s": round(step_bytes / median / 1e9, 1), "frac_hbm": round(step_bytes / median / 1e9 / (hbm_peak * world), 3),
              "distinct_first_tokens": len({t[0] for t in tokens}), "all_reduce": exchange,
              "decode_ms_per_step_by_exchange": exchange_ms or None}

    # (ii) one prefill of 4096 tokens, every position of the context
    runner = Qwen3Runner(weights, group=group, fused_allreduce=fused_allreduce)
    ws = Workspace(weights.config, full.context)
    ids = torch.tensor([int(t) for t in rng.integers(0, full.vocab, full.context)], dtype=torch.int32, device="cuda")
    times = []
    for _ in range(4):
        runner.control.zero_()
        if world > 1:
            dist.barrier(group)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        runner.forward(ws, ids)
        token = runner._read_next()
        times.append(time.perf_counter() - t0)
    if world > 1:
        slowest = torch.tensor(times, dtype=torch.float64, device="cuda")
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX, group=group)
        times = slowest.tolist()
    best = float(np.median(times[1:]))
    ops_total = 2.0 * full.context * (full.weight_bytes() - full.vocab * full.hidden) + 2.0 * full.vocab * full.hidden
    prefill = {"tokens": full.context, "ms": round(best * 1e3, 3), "tok_s": round(full.context / best, 1),
               "projection_TOPS": round(ops_total / best / 1e12, 1), "first_token": token,
               "all_reduce": "single GPU" if world == 1 else "NCCL all-reduce + residual kernel (4096 rows)"}
    del runner, ws
    torch.cuda.empty_cache()
    return {"workload": "configs[4]: 64 ragged sequences decoded side by side; one 4096-token prefill",
            "parallelism": f"tp{world}" if world > 1 else "single",
            "ragged_decode": ragged, "prefill_4096": prefill}


def cpu_step(oracle, host, threads):
    for M in DECODE_M:
        for name, K, N in SHAPES:
            x, w, ws = host[(M, name)]
            q, s = oracle.quantize(x)
            oracle.linear(q, s, w, ws, threads=threads)


def host_copies(torch, mats, bufs):
    host = {}
    wh = {name: (m.w.cpu().numpy(), m.scale.cpu().numpy()) for name, m in mats.items()}
    for (M, name), b in bufs.items():
        host[(M, name)] = (b["x"].float().cpu().numpy().copy(), *wh[name])
    return host


def cpu_baseline(torch, mats, bufs, reps):
    from oracle import oracle
    host = host_copies(torch, mats, bufs)
    threads = oracle.hw_threads()
    cpu_step(oracle, host, threads)
    t = time.perf_counter()
    for _ in range(reps):
        cpu_step(oracle, host, threads)
    dt = (time.perf_counter() - t) / reps
    nbytes = sum(linear_bytes(M, K, N) + quant_bytes(M, K) for M in DECODE_M for _, K, N in SHAPES)
    out = {"value": round(nbytes / dt / 1e9, 2), "unit": "GB/s", "cores": threads, "kind": "port",
           "sample": f"{reps} full steps (all 15 quantize+linear pairs) of the same workload, {threads} host threads",
           "s_per_step": round(dt, 4)}
    out["torch_path"] = torch_cpu_path(torch, host)
    return out


def torch_cpu_path(torch, host, budget_s=12.0):
    """The same path written as the reference's fixture generator writes it (tools/operator_fixtures.py:42-44,54):
    scale = amax/127, q = round(x/scale).clamp(+-127), out = bf16((q.int() @ w.int().T).float() * a_scale * w_scale), with
    torch.set_num_threads(8) (:17).  Torch's CPU int32 matmul is slow, so the (M, projection) pairs are timed one by one
    in the order of the workload until the time budget is spent; the figure is algorithmic bytes over time for the pairs
    that ran."""
    before = torch.get_num_threads()
    torch.set_num_threads(8)
    done_bytes, spent, ran = 0, 0.0, []
    try:
        for M in DECODE_M:
            for name, K, N in SHAPES:
                if spent > budget_s:
                    break
                x, w, ws = host[(M, name)]
                xt, wt, wst = torch.from_numpy(x), torch.from_numpy(w).int(), torch.from_numpy(ws)
                t = time.perf_counter()
                scale = xt.abs().amax(-1, keepdim=True).clamp(min=1e-8) / 127
                q = torch.round(xt / scale).clamp(-127, 127).to(torch.int8)
                out = ((q.int() @ wt.T).float() * scale * wst).bfloat16()
                spent += time.perf_counter() - t
                done_bytes += linear_bytes(M, K, N) + quant_bytes(M, K)
                ran.append(f"{name}@{M}")
                del out
    finally:
        torch.set_num_threads(before)
    return {"value": round(done_bytes / max(spent, 1e-9) / 1e9, 3), "unit": "GB/s", "cores": 8, "kind": "reference formula in torch (CPU)",
            "sample": f"{len(ran)} of 15 (M, projection) pairs within {budget_s:.0f} s: " + " ".join(ran), "seconds": round(spent, 2)}


def run_reference(args):
    """The reference's CPU-integer path (tools/operator_fixtures.py:43-44,54), restated in C (oracle/), on all host threads."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    from oracle import oracle
    threads = oracle.hw_threads()
    rng = np.random.default_rng(0)
    host = {}
    wh = {}
    for name, K, N in SHAPES:
        # uniform int8 codes: the integer product's speed does not depend on the value distribution
        w = rng.integers(-127, 128, (N, K), dtype=np.int8)
        wh[name] = (w, (rng.random(N, dtype=np.float32) * 1e-3 + 1e-4).astype(np.float32))
    for M in DECODE_M:
        for name, K, N in SHAPES:
            x = oracle.bf16(rng.standard_normal((M, K), dtype=np.float32))
            x[:, rng.choice(K, 8, replace=False)] *= 20
            host[(M, name)] = (oracle.bf16(x), *wh[name])
    t = time.perf_counter()
    cpu_step(oracle, host, threads)  # the first of the W warm-up steps
    first = time.perf_counter() - t
    # W warm-up and K timed steps as asked, unless that would take more than a few minutes on this host
    args.warmup = max(1, min(args.warmup, int(30 / first)))
    args.steps = max(1, min(args.steps, int(150 / first)))
    for _ in range(args.warmup - 1):
        cpu_step(oracle, host, threads)
    t = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(oracle, host, threads)
    dt = (time.perf_counter() - t) / args.steps
    nbytes = sum(linear_bytes(M, K, N) + quant_bytes(M, K) for M in DECODE_M for _, K, N in SHAPES)
    v = round(nbytes / dt / 1e9, 2)
    sample = f"full step (all 15 quantize+linear pairs), {threads} host threads, C restatement of the reference's CPU-integer path"
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": "GB/s", "n_gpus": args.gpus,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
                      "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
                      "dtype": "int8xint8->int32 (bf16 in/out)", "data": "synthetic",
                      "config": workload_config(args.gpus),
                      "execution": {"launch": "host threads", "all_reduce": "none", "all_reduce_check": None, "weight_copies": 1},
                      "cpu_baseline": {"value": v, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
                      "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-pdl", action="store_true", help="ordinary launches instead of programmatic dependent launches")
    ap.add_argument("--peer-allreduce", action="store_true",
                    help="tensor parallel, with --nccl-allreduce: the library's stand-alone one-shot peer-memory all-reduce instead "
                         "of NCCL (measured 3 us per call slower than NCCL at 2 and 4 GPUs)")
    ap.add_argument("--fused-max-ranks", type=int, default=8,
                    help="largest tensor-parallel degree that uses the fused exchange by default (it is checked bit for bit against "
                         "gathered partial sums before anything is timed; every rank falls back to NCCL together if the check fails)")
    ap.add_argument("--nccl-allreduce", dest="fused_allreduce", action="store_false",
                    help="tensor parallel: projection + NCCL all-reduce for O and down instead of w8a8_linear_allreduce (GEMV "
                         "epilogue pushes tagged packets to every rank, a consumer kernel sums them; the default: 0.286 against "
                         "0.319 ms per step at 2 GPUs)")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of CUDA-graph replays")
    ap.add_argument("--no-extra", action="store_true", help="skip the per-shape and prefill tables")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-model", action="store_true", help="skip the whole-model generation table")
    ap.add_argument("--shapes", default="", help="comma-separated subset of the five projections (profiling runs)")
    ap.add_argument("--ms", default="", help="comma-separated subset of the token counts (profiling runs)")
    ap.add_argument("--variant", type=int, default=0, help="force a kernel variant for every linear call (A/B runs)")
    ap.add_argument("--prefill-variant", type=int, default=0, help="force a kernel variant in the prefill table (A/B runs)")
    ap.add_argument("--prefill-ms", default="", help="comma-separated token counts of the prefill table (profiling runs)")
    args = ap.parse_args()
    global SHAPES, DECODE_M, PREFILL_M, WORKLOAD
    if args.prefill_ms:
        PREFILL_M = [int(m) for m in args.prefill_ms.split(",")]
    if args.shapes:
        keep = args.shapes.split(",")
        SHAPES = [s for s in SHAPES if s[0] in keep]
        WORKLOAD += f" [subset: shapes={args.shapes}]"
    if args.ms:
        DECODE_M = [int(m) for m in args.ms.split(",")]
        WORKLOAD += f" [subset: M={args.ms}]"
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
