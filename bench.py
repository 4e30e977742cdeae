#!/usr/bin/env python
"""Flagship benchmark: data-parallel training of a GPT-style 1.3 B decoder (24 layers, d=2048,
16 heads, sequence 2048, vocabulary 50257, bf16, uniform random token ids) with bucketed 25 MB
gradient reduce-scatter fused with scale/cast and overlapped with backward, sharded AdamW and
parameter all-gather -- tokens/s of the whole job.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3

Rank 0 prints one JSON line.  `value` is timed on the device (CUDA events, max over ranks) with the
batch already resident; `e2e` repeats the measurement through the public API with, every step, the
host->device copy of that step's token ids from pinned memory and a device->host read of the loss.
The same line carries
  * `baseline_ddp`: the same model, batch and step count in plain PyTorch (torch.nn + DistributedDataParallel with
    25 MB buckets + fused AdamW: NCCL, cuBLAS, cuDNN) measured in the same launch right after the framework's own
    steps; `vs_baseline` is value / the recorded tokens/s of that baseline on this GPU pool (same N);
  * `headline` (N >= 2): this library's headline metric -- all-reduce / reduce-scatter / all-gather bus GB/s at
    1 MB .. 1 GB with algo="auto" next to NCCL, and the fused tensor-parallel all-gather+GEMM and
    GEMM+reduce-scatter kernels next to NCCL+cuBLAS (sequential and stream-overlapped) at TP = N.
`--impl ddp` times only the PyTorch baseline and prints it in the same format.
`--impl reference` reports that the reference (napplesty/pccl) cannot be built or run.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def reference_arm() -> None:
    why = ("reference napplesty/pccl does not build: all 7 submodules are empty (nlohmann/json, asio, spdlog headers "
           "missing), infiniband/verbs.h absent, declaration/definition mismatches, and Engine::exeOp and the "
           "registry/buffer/operator managers have no definitions; it contains no kernel and no model to time")
    probe = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(probe) and os.listdir(probe):
        why += " (a partial install exists under baseline/_ref but exposes no runnable path)"
    if int(os.environ.get("RANK", "0")) == 0:          # one line per job, also under torch.distributed.run
        print(json.dumps({"impl": "reference", "unavailable": why}))


def ddp_arm(args, rank: int, world: int, local: int) -> None:
    """The PyTorch baseline alone, in the framework's output format (impl = "ddp")."""
    import torch
    import torch.distributed as dist
    from pccl_b200.baselines.ddp_gpt import measure
    from pccl_b200.models import GPTConfig
    from pccl_b200.utils import ClockSampler
    cfg = GPTConfig.gpt_1p3b() if args.model == "gpt-1.3b" else GPTConfig.tiny()
    sampler = ClockSampler(local).start()
    r = measure(cfg, world, rank, local, args.batch, args.steps, args.warmup, precision=args.ddp_precision, zero=args.ddp_zero)
    clocks = sampler.stop()
    if rank == 0:
        print(json.dumps({
            "impl": "ddp", "metric": "tokens/s, data-parallel GPT-1.3B training in plain PyTorch (DistributedDataParallel, "
            "25 MB buckets, fused AdamW)", "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"model": args.model, "params": r["params"], "global_batch": world * args.batch, "seq_len": cfg.seq_len,
                       "parallelism": f"dp{world}", "precision": r["precision"], "optimizer": r["optimizer"], "wrapper": r["wrapper"],
                       "l2": "no flush: each step streams >20 GB of weights/activations, far above the 126 MB L2"},
            "e2e": {"value": r.get("e2e_tokens_per_s"), "unit": "tokens/s", "ms_per_step": r.get("e2e_ms_per_step"),
                    "h2d_bytes_per_step": args.batch * (cfg.seq_len + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "model_tflops_per_gpu": cfg.flops_per_token() * r["tokens_per_s"] / world / 1e12,
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
            "final_loss": r["final_loss"]}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "ddp"])
    ap.add_argument("--ddp-precision", default="bf16", choices=["bf16", "amp"],
                    help="PyTorch baseline: bf16 parameters and optimizer state (fastest) or fp32 parameters under autocast")
    ap.add_argument("--ddp-zero", action="store_true", help="PyTorch baseline: ZeroRedundancyOptimizer around fused AdamW")
    ap.add_argument("--no-baseline", action="store_true", help="skip the in-launch PyTorch DDP baseline")
    ap.add_argument("--no-headline", action="store_true", help="skip the collective / fused-TP headline block at N > 1")
    ap.add_argument("--batch", type=int, default=int(os.environ.get("PCCL_BENCH_BATCH", "8")), help="sequences per GPU per step")
    ap.add_argument("--model", default="gpt-1.3b", choices=["gpt-1.3b", "tiny"])
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--comm-blocks", type=int, default=0, help="CTAs of the gradient/optimizer kernels (0 = automatic)")
    ap.add_argument("--algo", default="auto", choices=["auto", "nvls", "p2p"])
    ap.add_argument("--bucket-timing", action="store_true",
                    help="after the timed runs, one extra step with CUDA events around every gradient bucket's kernels (key dp_timing)")
    ap.add_argument("--unfused-blocks", action="store_true", help="every layer its own autograd node (comparison run)")
    ap.add_argument("--no-micro", action="store_true", help="skip the collective micro-benchmarks at N > 1")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N (N > 1) must be started with torch.distributed.run --nproc-per-node N")
        args.gpus = world
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=__import__("datetime").timedelta(seconds=180))

    if args.impl == "ddp":
        ddp_arm(args, rank, world, local)
        return

    from pccl_b200.engine import Engine
    from pccl_b200.models import GPT, GPTConfig
    from pccl_b200.ops import check_status, launch_count
    from pccl_b200.parallel import ShardedDataParallel
    from pccl_b200.utils import ClockSampler

    cfg = GPTConfig.gpt_1p3b() if args.model == "gpt-1.3b" else GPTConfig.tiny()
    cfg.fuse_blocks = not args.unfused_blocks
    torch.manual_seed(1234)            # same initial weights on every rank
    model = GPT(cfg, device="cuda")
    n_params = sum(p.numel() for p in model.parameters())
    os.environ.setdefault("PCCL_WORKSPACE_MB", "256")
    eng = Engine(rank, world)
    # gradient + parameter buckets (2 x 2 bytes per parameter), and room for the headline block's 1 GB collectives
    eng.initEngine("cuda", heap_bytes=max(int(4.4 * n_params) + (1 << 30), (3 << 30) if world > 1 else 0))
    if world > 1:
        eng.connect()
    heap_mark = eng.symmetric_mark()
    dp = ShardedDataParallel(model, eng, lr=1e-4, bucket_mb=args.bucket_mb, comm_blocks=args.comm_blocks, algo=args.algo)

    B, S = args.batch, cfg.seq_len
    total_steps = args.warmup + args.steps
    g = torch.Generator().manual_seed(1000 + rank)
    host_ids = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).pin_memory() for _ in range(total_steps)]
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident measurement ------------------------------------------------------------
    dev_batches = [h.cuda() for h in host_ids[:2]]
    for i in range(args.warmup):
        b = dev_batches[i % 2]
        dp.train_step(b[:, :-1], b[:, 1:])
    barrier()
    check_status("warm-up")
    sampler = ClockSampler(local).start()
    launches0 = launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = []
    e0.record()
    for i in range(args.steps):
        b = dev_batches[i % 2]
        loss = dp.train_step(b[:, :-1], b[:, 1:])
        if args.bucket_timing:                 # one more event per step: the per-step series goes into dp_timing
            marks.append(torch.cuda.Event(enable_timing=True))
            marks[-1].record()
    e1.record()
    barrier()
    dev_ms = max_over_ranks(e0.elapsed_time(e1))
    launches = launch_count() - launches0
    check_status("timed steps")
    final_loss = float(loss)

    # ---- end-to-end measurement: pinned H2D of the ids and D2H of the loss every step --------------
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    f0.record()
    for i in range(args.steps):
        ids = host_ids[args.warmup + i].to("cuda", non_blocking=True)
        loss = dp.train_step(ids[:, :-1], ids[:, 1:])
        loss_host.copy_(loss.reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()       # the user reads the loss every step
        _ = float(loss_host[0])
    f1.record()
    barrier()
    e2e_ms = max_over_ranks(f0.elapsed_time(f1))
    wall_ms = max_over_ranks((time.perf_counter() - t_wall) * 1e3)
    clocks = sampler.stop()
    check_status("end-to-end steps")

    grad_rs_schedule = dp.schedule
    dp_timing = None
    if args.bucket_timing:
        b = dev_batches[0]
        dp_timing = dp.timed_step(b[:, :-1], b[:, 1:])
        again = dp.timed_step(b[:, :-1], b[:, 1:])          # directly behind the first: no idle gap before it
        dp_timing["second_timed_step"] = {k: v for k, v in again.items() if k != "buckets"}
        prev = e0
        series = []
        for m in marks:
            series.append(prev.elapsed_time(m))
            prev = m
        dp_timing["step_ms_series"] = series
        mine = {"rank": rank, "forward_ms": dp_timing["forward_end"], "backward_ms": dp_timing["backward_end"] - dp_timing["forward_end"],
                "sm_mhz": clocks["sm_mhz"], "step_ms_mean": sum(series) / max(1, len(series))}
        if world > 1:
            every = [None] * world
            dist.all_gather_object(every, mine)
            dp_timing["ranks"] = every
        else:
            dp_timing["ranks"] = [mine]
        barrier()
    # ---- the library's headline metric and the PyTorch baseline, in the same launch -----------------------
    # The training state is released first: its buckets give the symmetric heap back to the 1 GB collectives,
    # and the baseline gets the device memory.
    del dp, model, dev_batches, loss
    import gc
    gc.collect()                      # the wrapper's hook closures form cycles
    torch.cuda.empty_cache()
    eng.symmetric_reset(heap_mark)
    head = None
    if world > 1 and not args.no_headline and not args.no_micro:
        try:
            from pccl_b200.bench_headline import headline
            head = headline(eng)
        except Exception as e:  # noqa: BLE001 - the training number must still be printed
            head = {"error": f"{type(e).__name__}: {e}"}
    baseline = None
    if not args.no_baseline:
        try:
            from pccl_b200.baselines.ddp_gpt import measure
            baseline = measure(cfg, world, rank, local, B, min(args.steps, 10), 3, precision=args.ddp_precision, e2e=False)
        except Exception as e:  # noqa: BLE001
            baseline = {"error": f"{type(e).__name__}: {e}"}

    from pccl_b200.baselines.ddp_gpt import recorded
    recorded_ddp = recorded(world) if args.model == "gpt-1.3b" and B == 8 else None
    tokens = world * B * S * args.steps
    value = tokens / (dev_ms / 1e3)
    e2e_value = tokens / (max(e2e_ms, wall_ms) / 1e3)
    flops = cfg.flops_per_token() * tokens / (dev_ms / 1e3)
    if rank == 0:
        out = {
            "metric": "tokens/s, data-parallel GPT-1.3B training (bf16, 25 MB gradient buckets, reduce-scatter fused "
                      "with scale/cast and overlapped with backward)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / recorded_ddp) if recorded_ddp else (
                value / baseline["tokens_per_s"] if baseline and baseline.get("tokens_per_s") else None),
            "vs_baseline_source": ("recorded PyTorch DDP tokens/s for this N on this GPU pool" if recorded_ddp else
                                   ("PyTorch DDP measured in this launch (no recorded number for this N)"
                                    if baseline and baseline.get("tokens_per_s") else None)),
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init weights)",
            "config": {"model": "gpt-1.3b (24 layers, d=2048, 16 heads, vocab 50257)" if args.model == "gpt-1.3b" else "tiny",
                       "params": n_params, "global_batch": world * B, "seq_len": S, "parallelism": f"dp{world}",
                       "bucket_mb": args.bucket_mb, "optimizer": "sharded AdamW (ZeRO-1) + parameter all-gather",
                       "transport": "nvls" if eng.has_nvls else ("p2p" if world > 1 else "local"),
                       "grad_rs_schedule": grad_rs_schedule,
                       "l2": "no flush: each step streams >20 GB of weights/activations, far above the 126 MB L2"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": max(e2e_ms, wall_ms) / args.steps,
                    "h2d_bytes_per_step": B * (S + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "model_tflops_per_gpu": flops / world / 1e12,
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
            "final_loss": final_loss,
        }
        out["baseline"] = {"what": "PyTorch DistributedDataParallel (NCCL, 25 MB buckets) + cuBLAS/cuDNN eager model + fused AdamW, "
                                   "same model, batch and sequence length, on this GPU pool", "recorded_tokens_per_s": recorded_ddp,
                           "source": "pccl_b200/baselines/ddp_gpt1p3b_b200.json (bench.py --impl ddp)"}
        if baseline is not None:
            out["baseline_ddp"] = baseline
            if "tokens_per_s" in baseline:
                out["baseline_ddp"]["ratio_ours_over_ddp_same_launch"] = value / baseline["tokens_per_s"]
        if dp_timing is not None:
            out["dp_timing"] = dp_timing
        if head is not None:
            out["headline"] = head
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
    del eng          # unbind and unmap the symmetric heap while every rank is still here
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
