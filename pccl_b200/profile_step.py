"""Per-kernel breakdown of one data-parallel training step of the GPT model on one GPU.

    python -m pccl_b200.profile_step --batch 8 --steps 2 --out step_profile.txt

Runs a few warm-up steps, then records ``--steps`` steps with the PyTorch profiler (CUPTI kernel
activity) and writes the kernels sorted by device time: name, total and mean microseconds, calls and
share of the step.  It answers "which kernels make up the step, and which of them are still library
or eager PyTorch kernels" -- the list that fusion work is planned from.  The timings are taken under
a profiler, so they rank kernels; they are not benchmark numbers.
"""
from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--model", default="gpt-1.3b", choices=["gpt-1.3b", "tiny"])
    ap.add_argument("--rows", type=int, default=40)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    from torch.profiler import ProfilerActivity, profile

    from .engine import Engine
    from .models import GPT, GPTConfig
    from .parallel import ShardedDataParallel
    cfg = GPTConfig.gpt_1p3b() if args.model == "gpt-1.3b" else GPTConfig.tiny()
    torch.manual_seed(0)
    model = GPT(cfg, device="cuda")
    n = sum(p.numel() for p in model.parameters())
    eng = Engine(0, 1)
    eng.initEngine("cuda", heap_bytes=int(4.4 * n) + (1 << 30))
    dp = ShardedDataParallel(model, eng, lr=1e-4)
    ids = torch.randint(0, cfg.vocab_size, (args.batch, cfg.seq_len + 1), device="cuda")
    for _ in range(3):
        dp.train_step(ids[:, :-1], ids[:, 1:])
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(args.steps):
            dp.train_step(ids[:, :-1], ids[:, 1:])
        torch.cuda.synchronize()
    rows = [(e.key, e.device_time_total, e.count) for e in prof.key_averages() if e.device_time_total > 0]
    rows.sort(key=lambda r: -r[1])
    total = sum(r[1] for r in rows)
    lines = [f"# one training step, {args.model}, batch {args.batch} x {cfg.seq_len}, one GPU; kernel time summed over {args.steps} steps",
             f"# total kernel time per step: {total / args.steps / 1e3:.2f} ms",
             f"{'share':>6} {'us/step':>10} {'calls/step':>10} {'mean us':>9}  kernel"]
    for name, t, c in rows[:args.rows]:
        lines.append(f"{100 * t / total:6.2f} {t / args.steps:10.1f} {c / args.steps:10.1f} {t / c:9.1f}  {name[:150]}")
    rest = sum(r[1] for r in rows[args.rows:])
    lines.append(f"{100 * rest / total:6.2f} {rest / args.steps:10.1f} {'':>10} {'':>9}  ({len(rows) - args.rows} more kernels)")
    text = "\n".join(lines)
    print(text)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text + "\n")


if __name__ == "__main__":
    main()
