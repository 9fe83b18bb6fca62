"""Where one training step of the GPT-2 124M benchmark spends its device time.

Runs the same model, data and optimizer settings as ``bench.py`` on one GPU and brackets the
three phases of every step with CUDA events:

  forward    autocast bf16 forward + loss
  backward   loss.backward()
  optimizer  optimizer.step() + zero_grad()

The host is synchronised only once, after the last step, so that it runs ahead of the device
as it does in ``bench.py``; the events then split the device timeline of each step.

    python benchmarks/step_breakdown.py --impl ours --steps 10
    python benchmarks/step_breakdown.py --impl reference --steps 10

Prints one JSON line with the median milliseconds of each phase.  Shares, not a headline number.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)

import bench  # noqa: E402  (the benchmark's model and optimizer builders)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--backend", default="native")
    ap.add_argument("--gemm-mode", default="tf32x3")
    ap.add_argument("--comm", default="p2p")
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--batch", type=int, default=bench.BATCH_PER_GPU)
    ap.add_argument("--model", choices=["fused", "plain"], default="fused")
    ap.add_argument("--kernel-table", type=int, default=0, metavar="ROWS",
                    help="also run 3 steps under torch.profiler and print the ROWS kernels with the most device time")
    args = ap.parse_args()

    import torch

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(1234)
    torch.backends.cuda.matmul.allow_tf32 = False
    if args.impl == "ours" and args.model == "fused":
        from optimizers_b200.models import GPT2, GPT2Config

        model = GPT2(GPT2Config(n_layer=args.layers)).to(dev)
    else:
        model = bench.make_gpt2(args.layers).to(dev)
    opt = bench.build_optimizer(args.impl, model, 1, args)
    gen = torch.Generator().manual_seed(100)
    tokens = [torch.randint(0, bench.VOCAB, (args.batch, bench.SEQ + 1), generator=gen).to(dev) for _ in range(4)]

    def ev():
        return torch.cuda.Event(enable_timing=True)

    phases: dict[str, list[float]] = {"forward": [], "backward": [], "optimizer": [], "step": []}
    marks = []
    for i in range(args.warmup + args.steps):
        t = tokens[i % 4]
        e0, e1, e2, e3 = ev(), ev(), ev(), ev()
        e0.record()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(t[:, :-1], t[:, 1:])
        e1.record()
        loss.backward()
        e2.record()
        opt.step()
        opt.zero_grad(set_to_none=True)
        e3.record()
        if i == 0:
            torch.cuda.synchronize()  # the first step holds the long root-inverse refresh
        if i >= args.warmup:
            marks.append((e0, e1, e2, e3))
    torch.cuda.synchronize()
    for e0, e1, e2, e3 in marks:
        phases["forward"].append(e0.elapsed_time(e1))
        phases["backward"].append(e1.elapsed_time(e2))
        phases["optimizer"].append(e2.elapsed_time(e3))
        phases["step"].append(e0.elapsed_time(e3))
    out = {"impl": args.impl, "steps": args.steps, "batch": args.batch, "seq_len": bench.SEQ}
    out.update({f"{k}_ms": round(statistics.median(v), 3) for k, v in phases.items()})
    print(json.dumps(out))
    if args.kernel_table:
        from torch.profiler import profile, ProfilerActivity

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(3):
                t = tokens[i % 4]
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss = model(t[:, :-1], t[:, 1:])
                loss.backward()
                opt.step()
                opt.zero_grad(set_to_none=True)
            torch.cuda.synchronize()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.kernel_table, max_name_column_width=90))


if __name__ == "__main__":
    main()
