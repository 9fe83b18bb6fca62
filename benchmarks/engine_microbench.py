"""Optimizer-only benchmark through the public API: ``--blocks`` parameters of size d x d, fp32,
gradients N(0, 1e-2), one ``optimizer.step()`` per iteration, timed with CUDA events.

Two numbers per run:

  step_ms      median time of a step that does not recompute the preconditioners (gradient
               prologue, factor update, preconditioner application, epilogue)
  refresh_ms   median extra time of a step that does (root inverse by eigendecomposition or by the
               coupled Newton iteration, or the eigenbasis refresh of the eigenvalue-corrected
               variant), measured as refresh step - plain step

``--impl reference`` runs the unmodified reference package from ``baseline/_ref`` with the same
settings, for comparison on the same GPU.

    python benchmarks/engine_microbench.py --d 2048 --blocks 16 --root eigen
    python benchmarks/engine_microbench.py --d 1024 --blocks 64 --root newton --impl reference
    python benchmarks/engine_microbench.py --optimizer gpa --d 4096 --blocks 16
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/engine_microbench.py --dim 2048 --blocks 64 --comm p2p      # block work split over 8 ranks
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--optimizer", choices=["shampoo", "soap", "gpa"], default="shampoo")
    ap.add_argument("--root", choices=["eigen", "newton"], default="eigen")
    ap.add_argument("--eigenbasis", choices=["eigh", "qr"], default="eigh", help="refresh method of --optimizer soap")
    ap.add_argument("--dim", "--d", dest="d", type=int, default=2048, help="block size (use --dim under torchrun, which claims --d)")
    ap.add_argument("--blocks", type=int, default=16)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--refreshes", type=int, default=2)
    ap.add_argument("--backend", default="native")
    ap.add_argument("--gemm-mode", default="tf32x3")
    ap.add_argument("--fuse-grads", action="store_true",
                    help="with --comm p2p: owners sum the peers' gradients inside the prologue kernel (the gradients "
                    "live in the peer-addressable arena)")
    ap.add_argument("--phases", action="store_true",
                    help="also print the device time between the phase boundaries of the native step (max over ranks) "
                    "and the bytes that cross NVLink per rank")
    ap.add_argument("--comm", choices=["nccl", "p2p"], default="nccl",
                    help="under torchrun (N > 1, DDP distributor, bf16 search directions): NCCL all-gather or the "
                    "epilogue's stores into every peer's gather buffer")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
        import distributed_shampoo as lib
    else:
        sys.path.insert(0, REPO)
        import optimizers_b200 as lib

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    d, nb = args.d, args.blocks
    params = [torch.nn.Parameter(torch.randn(d, d, device=dev) * 0.02) for _ in range(nb)]
    grads = [[torch.randn(d, d, device=dev) * 1e-2 for _ in range(nb)] for _ in range(2)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    period = 1000

    if args.optimizer == "gpa":
        if args.impl == "reference":
            # The reference's wheel ships distributed_shampoo only; its gpa package is copied beside it
            # (cp -r <reference>/gpa baseline/_ref/gpa), unmodified.
            if not os.path.isdir(os.path.join(REPO, "baseline", "_ref", "gpa")):
                raise SystemExit("baseline/_ref/gpa is missing: copy the reference's gpa package there")
            from gpa.gpa_adamw import GPAAdamW
        else:
            from optimizers_b200.gpa_adamw import GPAAdamW

        opt = GPAAdamW(params, lr=1e-3, weight_decay=1e-2)
        opt.train()
    else:
        extra = {}
        if args.impl == "ours":
            extra["native_runtime_config"] = lib.NativeRuntimeConfig(
                backend=args.backend, gemm_mode=args.gemm_mode, comm_path=args.comm if world > 1 else "nccl",
                fuse_gradient_reduction=args.fuse_grads and world > 1 and args.comm == "p2p",
            )
        if world > 1:
            extra["distributed_config"] = lib.DDPDistributedConfig(
                communication_dtype=torch.bfloat16, num_trainers_per_group=world
            )
        if args.optimizer == "soap":
            pc = lib.EigenvalueCorrectedShampooPreconditionerConfig(
                amortized_computation_config=lib.QREigendecompositionConfig()
                if args.eigenbasis == "qr" else lib.EighEigendecompositionConfig()
            )
        elif args.root == "newton":
            pc = lib.RootInvShampooPreconditionerConfig(amortized_computation_config=lib.CoupledNewtonConfig())
        else:
            pc = lib.RootInvShampooPreconditionerConfig()
        opt = lib.DistributedShampoo(
            params, lr=1e-3, betas=(0.9, 0.999), epsilon=1e-6, max_preconditioner_dim=max(d, 2048),
            precondition_frequency=period, start_preconditioning_step=period,
            grafting_config=lib.AdaGradPreconditionerConfig(epsilon=1e-10), preconditioner_config=pc, **extra,
        )
        # The shared step counter (a CPU tensor aliased under every parameter); preset so that the
        # first warm-up step is the first preconditioned one.
        step_counter = next(s["step"] for s in opt.state.values() if "step" in s)
        step_counter.fill_(period - 1)

    fused_grads = args.impl == "ours" and args.optimizer != "gpa" and args.fuse_grads and world > 1 and args.comm == "p2p"

    def one_step(i: int) -> float:
        for p, g in zip(params, grads[i % 2]):
            if fused_grads:
                p.grad.copy_(g)  # .grad is the parameter's view of the shared gradient arena
            else:
                p.grad = g
        flush.zero_()
        if world > 1:
            dist.barrier()  # ranks enter the step together
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        opt.step()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e)
        if world > 1:  # the slowest rank counts
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for i in range(3):
        one_step(i)
    plain = [one_step(i) for i in range(args.steps)]
    refresh: list[float] = []
    if args.optimizer != "gpa":
        for i in range(args.refreshes + 1):
            step_counter.fill_(period * (i + 2) - 1)  # the next step recomputes the preconditioners
            t = one_step(i)
            if i > 0:  # the first refresh also pays one-time set-up (workspaces, handles)
                refresh.append(t)
    step_ms = statistics.median(plain)
    out = {
        "impl": args.impl, "optimizer": args.optimizer,
        "root": args.root if args.optimizer == "shampoo" else (args.eigenbasis if args.optimizer == "soap" else None),
        "n_gpus": world, "comm": args.comm if world > 1 else None,
        "d": d, "blocks": nb, "step_ms": round(step_ms, 4),
        "refresh_ms": round(statistics.median(refresh) - step_ms, 3) if refresh else None,
        "bytes_param_state": nb * d * d * 4,
    }
    if args.impl == "ours" and args.optimizer != "gpa":
        eng = opt._per_group_state_lists[0].get("native_engine")
        out["native_launches_per_step"] = eng.launches_per_step if eng is not None else 0
    if args.phases and args.impl == "ours" and args.optimizer != "gpa":
        eng = opt._per_group_state_lists[0].get("native_engine")
        if eng is not None:
            samples: dict[str, list[float]] = {}
            for i in range(args.steps):
                eng.phase_events = []
                one_step(i)
                marks = eng.phase_events
                for (_, a), (name, b) in zip(marks, marks[1:]):
                    samples.setdefault(name, []).append(a.elapsed_time(b))
            eng.phase_events = None
            names = list(samples)
            med = torch.tensor([statistics.median(samples[n]) for n in names], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(med, op=dist.ReduceOp.MAX)
            out["phase_ms"] = {n: round(v, 4) for n, v in zip(names, med.tolist())}
            # NVLink bytes per rank and step: an owner pulls the other ranks' fp32 gradients of its blocks
            # and stores its bf16 directions into the other ranks' gather buffers
            owned = nb / world
            elems = owned * d * d
            out["nvlink_bytes_per_rank"] = {
                "gradient_pull_fp32": int(elems * 4 * (world - 1)) if fused_grads else 0,
                "direction_push_bf16": int(elems * 2 * (world - 1)) if (world > 1 and args.comm == "p2p") else 0,
            }
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
