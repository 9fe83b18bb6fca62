"""Throughput benchmark: GPT-2 124M training with Distributed Shampoo.

Metric: training tokens per second (whole job) and milliseconds per step, on N GPUs of one
node.  Model and optimizer follow the reference benchmark configuration: 12 layers,
d_model 768, 12 heads, MLP 3072, vocabulary 50257, sequence 1024, batch 16 per GPU, bf16
autocast, fp32 Kronecker factors, max_preconditioner_dim 2048, precondition_frequency 100,
AdaGrad grafting.  Data is synthetic (uniform token ids) and weights are randomly initialised.

    python bench.py --gpus 1 --steps 20 --warmup 5                  # this framework
    python bench.py --impl reference --gpus 1 --steps 20 --warmup 5 # unmodified reference
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

What is reported is what training costs per step once the preconditioner refresh is counted:

    amortized ms/step = steady ms/step + (refresh step ms - steady ms/step) / precondition_frequency

``steady`` is the device time of the K timed steps, none of which recomputes the inverse roots
(the step counter of the optimizer is preset to ``start_preconditioning_step - 1``, in both arms,
so that the first warm-up step performs the first refresh and every later step runs the
preconditioned path).  ``refresh step`` is one more step, timed on the device after the timed
regions with the counter set so that it recomputes every inverse root (the refresh of a run in
progress: allocator and kernels warm; the first, cold one is reported separately).  ``value`` is
tokens/s at the amortised step time.

Rank 0 prints one JSON line.  The K steps are timed on the device with CUDA events (inputs
already on the device); ``optimizer_step_ms`` is the device time of ``optimizer.step()`` inside
those steps; ``e2e`` repeats the K steps through the public API with a pinned-host -> device copy
of each step's tokens and a device -> host read of each step's loss inside the timed region and
is amortised the same way.  ``plain_model`` (this framework's arm only) repeats the steady
measurement with the plain PyTorch GPT-2 that the reference arm uses, which isolates the
optimizer's share of the difference between the arms.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(REPO, "baseline", "_ref")

SEQ = 1024
BATCH_PER_GPU = 16
VOCAB = 50257
MAX_PRECOND_DIM = 2048
PRECOND_FREQ = 100


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--backend", choices=["auto", "native", "torch"], default="native")
    ap.add_argument("--gemm-mode", choices=["tf32x3", "tf32"], default="tf32x3")
    ap.add_argument("--comm", choices=["p2p", "nccl"], default="p2p", help="multi-GPU path of this framework")
    ap.add_argument("--parallelism", choices=["ddp", "hsdp"], default="hsdp",
                    help="N > 1: the hybrid-sharded distributor over FSDP HYBRID_SHARD with a (N / min(N, 4)) x min(N, 4) "
                    "replicate x shard mesh (default: the benchmark configuration, 2 x 4 on eight GPUs) or the DDP distributor; "
                    "the other one is measured as well and reported under other_parallelism")
    ap.add_argument("--single-parallelism", action="store_true", help="N > 1: measure only --parallelism")
    ap.add_argument("--model", choices=["fused", "plain"], default="fused",
                    help="this framework's arm: its GPT-2 with the fused norm / LM-head-loss kernels, or the plain "
                    "PyTorch model that the reference arm always uses")
    ap.add_argument("--no-plain", action="store_true", help="skip the extra plain-model measurement of this framework's arm")
    ap.add_argument("--layers", type=int, default=12, help="debug only; the reported config needs 12")
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU, help="debug only; the reported config needs 16")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index: int) -> None:
        self.index = index
        self.proc: subprocess.Popen | None = None
        self.lines: list[str] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def make_gpt2(n_layer: int):
    """Plain-PyTorch GPT-2 124M (pre-LN, learned positions, tied embedding), defined here so that
    the reference arm imports nothing from this repository's package."""
    import math

    import torch
    import torch.nn as nn
    import torch.nn.functional as F

    d_model, n_head, d_mlp, n_ctx = 768, 12, 3072, 1024

    class Block(nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.ln_1 = nn.LayerNorm(d_model)
            self.attn_qkv = nn.Linear(d_model, 3 * d_model)
            self.attn_proj = nn.Linear(d_model, d_model)
            self.ln_2 = nn.LayerNorm(d_model)
            self.mlp_fc = nn.Linear(d_model, d_mlp)
            self.mlp_proj = nn.Linear(d_mlp, d_model)

        def forward(self, x):
            B, T, C = x.shape
            q, k, v = self.attn_qkv(self.ln_1(x)).split(C, dim=2)
            q, k, v = (t.view(B, T, n_head, C // n_head).transpose(1, 2) for t in (q, k, v))
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + self.attn_proj(a.transpose(1, 2).reshape(B, T, C))
            return x + self.mlp_proj(F.gelu(self.mlp_fc(self.ln_2(x)), approximate="tanh"))

    class GPT2(nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.wte = nn.Embedding(VOCAB, d_model)
            self.wpe = nn.Embedding(n_ctx, d_model)
            self.blocks = nn.ModuleList(Block() for _ in range(n_layer))
            self.ln_f = nn.LayerNorm(d_model)
            for m in self.modules():
                if isinstance(m, (nn.Linear, nn.Embedding)):
                    nn.init.normal_(m.weight, mean=0.0, std=0.02)
                if isinstance(m, nn.Linear):
                    nn.init.zeros_(m.bias)
            for name, p in self.named_parameters():
                if name.endswith("proj.weight"):
                    nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * n_layer))

        def forward(self, idx, targets):
            x = self.wte(idx) + self.wpe(torch.arange(idx.shape[1], device=idx.device))
            for blk in self.blocks:
                x = blk(x)
            logits = F.linear(self.ln_f(x), self.wte.weight)
            return F.cross_entropy(logits.view(-1, logits.size(-1)).float(), targets.reshape(-1))

    return GPT2()


def build_optimizer(impl: str, model, world: int, args, mesh=None):
    import torch

    if impl == "reference":
        sys.path.insert(0, REF_DIR)
        import distributed_shampoo as lib  # the unmodified reference, installed under baseline/_ref

        assert os.path.realpath(lib.__file__).startswith(os.path.realpath(REF_DIR)), lib.__file__
        extra = {}
    else:
        import optimizers_b200 as lib

        p2p = world > 1 and args.comm == "p2p" and args.backend != "torch"
        extra = {
            "native_runtime_config": lib.NativeRuntimeConfig(
                backend=args.backend, gemm_mode=args.gemm_mode, comm_path="p2p" if p2p else "nccl",
                # DDP: owners pull and sum the peers' gradients in the prologue kernel; under HSDP the
                # FSDP wrapper has already reduced them, only the all-gather of the directions is fused
                fuse_gradient_reduction=p2p and mesh is None,
            )
        }
    if mesh is not None:
        dist_cfg = lib.HSDPDistributedConfig(
            param_to_metadata=lib.compile_fsdp_parameter_metadata(model), device_mesh=mesh,
            communication_dtype=torch.bfloat16, num_trainers_per_group=-1,
        )
    elif world > 1:
        dist_cfg = lib.DDPDistributedConfig(communication_dtype=torch.bfloat16, num_trainers_per_group=world)
    else:
        dist_cfg = lib.DefaultSingleDeviceDistributedConfig
    opt = lib.DistributedShampoo(
        model.parameters(),
        lr=1e-3,
        betas=(0.9, 1.0),
        epsilon=1e-12,
        max_preconditioner_dim=MAX_PRECOND_DIM,
        precondition_frequency=PRECOND_FREQ,
        start_preconditioning_step=PRECOND_FREQ,
        grafting_config=lib.AdaGradPreconditionerConfig(epsilon=1e-10),
        distributed_config=dist_cfg,
        **extra,
    )
    # Resume-style preset of the shared step counter (a CPU tensor aliased under every parameter).
    for state in opt.state.values():
        if "step" in state:
            state["step"].fill_(PRECOND_FREQ - 1)
            break
    return opt


def count_native_launches(opt) -> int:
    total = 0
    for rec in getattr(opt, "_per_group_state_lists", []):
        eng = rec.get("native_engine") if isinstance(rec, dict) else None
        if eng is not None:
            total += eng.launches_per_step
    return total


def main() -> None:
    args = parse_args()
    if args.impl == "reference" and not os.path.isdir(os.path.join(REF_DIR, "distributed_shampoo")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is missing; install the reference with pip --target baseline/_ref"}))
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # Convenience: re-launch under torchrun when called as plain `python bench.py --gpus N`.
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.abspath(__file__), *sys.argv[1:]]
            raise SystemExit(subprocess.call(cmd))
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    if args.impl == "ours":
        sys.path.insert(0, REPO)
    torch.manual_seed(1234)
    torch.backends.cuda.matmul.allow_tf32 = False  # optimizer math of the reference stays fp32
    fused_model = args.impl == "ours" and args.model == "fused"
    p2p_requested = args.impl == "ours" and world > 1 and args.comm == "p2p" and args.backend != "torch"

    def run_arm(parallelism: str, with_plain: bool) -> dict:
        """Build model + optimizer under one parallelism, measure, and return the figures (maxima
        over ranks)."""
        hsdp = world > 1 and parallelism == "hsdp"
        fused_comm = p2p_requested and not hsdp

        def build(use_fused_model: bool):
            """Model, its training wrapper and the optimizer of one arm."""
            if use_fused_model:
                # Same architecture, initialisation and autocast numerics as make_gpt2; the normalisations
                # and the LM head + cross-entropy run through this framework's CUDA kernels.
                from optimizers_b200.models import GPT2, GPT2Config

                model = GPT2(GPT2Config(n_layer=args.layers)).to(dev)
            else:
                model = make_gpt2(args.layers).to(dev)
            train_model = model
            mesh = None
            # This framework's p2p path reduces the gradients inside the optimizer's prologue kernel
            # (owners pull their blocks from peer memory), so the model is not wrapped in DDP there.
            if hsdp:
                from torch.distributed.device_mesh import init_device_mesh
                from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, ShardingStrategy

                shard = min(world, 4)
                mesh = init_device_mesh("cuda", (world // shard, shard), mesh_dim_names=("replicate", "shard"))
                train_model = model = FSDP(
                    model, device_mesh=mesh, sharding_strategy=ShardingStrategy.HYBRID_SHARD, use_orig_params=True,
                    device_id=local_rank,
                )
            elif world > 1 and not fused_comm:
                train_model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank])
            elif world > 1:
                for p in model.parameters():
                    dist.broadcast(p.data, src=0)
            opt = build_optimizer(args.impl, model, world, args, mesh)
            if hasattr(opt, "train"):
                opt.train()
            return train_model, opt

        B = args.batch
        gen = torch.Generator().manual_seed(100 + rank)
        n_batches = 8
        host_tokens = [torch.randint(0, VOCAB, (B, SEQ + 1), generator=gen).pin_memory() for _ in range(n_batches)]
        dev_tokens = [t.to(dev) for t in host_tokens]

        def barrier() -> None:
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def set_step_counter(opt, value: int) -> None:
            # Resume-style preset of the shared step counter (a CPU tensor aliased under every parameter).
            for state in opt.state.values():
                if "step" in state:
                    state["step"].fill_(value)
                    break

        def measure(train_model, opt, steps: int, warmup: int, with_refresh: bool) -> dict:
            opt_start = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
            opt_stop = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]

            def train_step(tokens: torch.Tensor, k: int | None = None) -> torch.Tensor:
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss = train_model(tokens[:, :-1], tokens[:, 1:])
                loss.backward()
                if k is not None:
                    opt_start[k].record()
                opt.step()
                if k is not None:
                    opt_stop[k].record()
                opt.zero_grad(set_to_none=not fused_comm)
                return loss

            # ---- warm-up (untimed); the first step performs the first (cold) refresh
            first_ms = None
            for i in range(max(warmup, 1)):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                train_step(dev_tokens[i % n_batches])
                torch.cuda.synchronize()
                if i == 0:
                    first_ms = (time.perf_counter() - t0) * 1e3

            # ---- device-timed region: K steps, inputs resident on the device
            barrier()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(steps):
                train_step(dev_tokens[i % n_batches], i)
            stop.record()
            barrier()
            out = {
                "first_step_ms": first_ms,
                "steady_ms": start.elapsed_time(stop) / steps,
                "optimizer_ms": sum(a.elapsed_time(b) for a, b in zip(opt_start, opt_stop)) / steps,
            }
            if not with_refresh:
                return out

            # ---- end-to-end region: pinned host tokens in, loss out, every step
            barrier()
            h2d = d2h = 0
            e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t_wall = time.perf_counter()
            e_start.record()
            last = 0.0
            for i in range(steps):
                src = host_tokens[i % n_batches]
                tokens = src.to(dev, non_blocking=True)
                h2d += src.numel() * src.element_size()
                loss = train_step(tokens)
                last = loss.item()
                d2h += loss.element_size()
            e_stop.record()
            barrier()
            out["e2e_ms"] = max(e_start.elapsed_time(e_stop), (time.perf_counter() - t_wall) * 1e3 if world == 1 else 0.0) / steps
            out["h2d"], out["d2h"], out["final_loss"] = h2d // max(steps, 1), d2h // max(steps, 1), last

            # ---- one refresh step of the run in progress (every inverse root recomputed), device-timed
            set_step_counter(opt, 3 * PRECOND_FREQ - 1)
            barrier()
            r_start, r_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r_start.record()
            train_step(dev_tokens[0])
            r_stop.record()
            barrier()
            out["refresh_ms"] = r_start.elapsed_time(r_stop)
            return out

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        train_model, opt = build(fused_model)
        model_launches = 0
        if fused_model:
            from optimizers_b200.models import fused_ops

            model_launches = -fused_ops.launch_count
        m = measure(train_model, opt, args.steps, args.warmup, with_refresh=True)
        if fused_model:
            # launches of the model kernels per step, from the whole measured run
            steps_run = max(args.warmup, 1) + 2 * args.steps + 1
            model_launches = (model_launches + fused_ops.launch_count) // steps_run
        clocks = sampler.stop() if rank == 0 else {}
        launches_per_step = (count_native_launches(opt) + model_launches) if args.impl == "ours" else 0

        plain = None
        if with_plain and args.impl == "ours" and fused_model and not args.no_plain:
            del train_model, opt
            torch.cuda.empty_cache()
            torch.manual_seed(1234)
            plain_model, plain_opt = build(False)
            plain = measure(plain_model, plain_opt, args.steps, args.warmup, with_refresh=False)
            del plain_model, plain_opt

        keys = ["steady_ms", "optimizer_ms", "e2e_ms", "refresh_ms", "first_step_ms"]
        times = torch.tensor([m[k] for k in keys] + ([plain["steady_ms"], plain["optimizer_ms"]] if plain else [0.0, 0.0]),
                             device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
        steady_ms, optimizer_ms, e2e_ms, refresh_ms, first_ms, plain_ms, plain_opt_ms = times.tolist()

        def amortized(step_ms: float) -> float:
            return step_ms + max(refresh_ms - steady_ms, 0.0) / PRECOND_FREQ

        tokens_per_step = B * SEQ * world
        value = tokens_per_step / (amortized(steady_ms) / 1e3)
        e2e_value = tokens_per_step / (amortized(e2e_ms) / 1e3)
        tokens = B * SEQ * world
        return {
            "hsdp": hsdp, "fused_comm": fused_comm, "steady_ms": steady_ms, "optimizer_ms": optimizer_ms, "e2e_ms": e2e_ms,
            "refresh_ms": refresh_ms, "first_ms": first_ms, "plain": (plain_ms, plain_opt_ms) if plain is not None else None,
            "amortized_ms": amortized(steady_ms), "e2e_amortized_ms": amortized(e2e_ms),
            "value": tokens / (amortized(steady_ms) / 1e3), "e2e_value": tokens / (amortized(e2e_ms) / 1e3),
            "final_loss": m["final_loss"], "h2d": m["h2d"], "d2h": m["d2h"], "clocks": clocks,
            "launches_per_step": launches_per_step, "batch": B,
        }

    def describe(r: dict) -> tuple[str, str]:
        if world == 1:
            return "single", "none"
        if r["hsdp"]:
            par = f"hsdp{world} (replicate {world // min(world, 4)} x shard {min(world, 4)})"
            comm = ("FSDP reduce-scatter (NCCL); directions all-gathered over the replicate group by peer stores fused into the epilogue kernel"
                    if p2p_requested else "nccl")
        else:
            par = f"dp{world}"
            comm = "p2p fused reduce-scatter + all-gather kernels" if r["fused_comm"] else "nccl"
        return par, comm

    main_par = args.parallelism if world > 1 else "ddp"
    r = run_arm(main_par, with_plain=True)
    other = None
    if world > 1 and not args.single_parallelism:
        other = run_arm("ddp" if main_par == "hsdp" else "hsdp", with_plain=False)
    B = r["batch"]
    value, e2e_value = r["value"], r["e2e_value"]
    steady_ms, optimizer_ms, e2e_ms, refresh_ms, first_ms = (r[k] for k in ("steady_ms", "optimizer_ms", "e2e_ms", "refresh_ms", "first_ms"))
    clocks, launches_per_step, hsdp, fused_comm = r["clocks"], r["launches_per_step"], r["hsdp"], r["fused_comm"]
    plain = r["plain"]
    plain_ms, plain_opt_ms = plain if plain is not None else (0.0, 0.0)
    m = {"final_loss": r["final_loss"], "h2d": r["h2d"], "d2h": r["d2h"]}

    def amortized(step_ms: float) -> float:
        return step_ms + max(refresh_ms - steady_ms, 0.0) / PRECOND_FREQ

    if rank == 0:
        out = {
            "metric": "train tokens/sec (GPT-2 124M, Distributed Shampoo), preconditioner refresh amortised over precondition_frequency steps",
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": amortized(steady_ms),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init weights",
            "impl": args.impl,
            "config": {
                "model": f"gpt2-124m ({args.layers} layers, d_model 768, 12 heads, mlp 3072, vocab 50257)",
                "model_impl": "framework GPT-2: fused LayerNorm and LM-head cross-entropy kernels" if fused_model
                else "plain PyTorch modules",
                "global_batch": B * world,
                "seq_len": SEQ,
                "parallelism": describe(r)[0],
                "comm": describe(r)[1],
                "optimizer": "DistributedShampoo max_preconditioner_dim=2048 precondition_frequency=100 AdaGrad grafting, fp32 factors",
                "gemm_mode": args.gemm_mode if args.impl == "ours" else "fp32 (cuBLAS)",
                "l2_policy": "working set (params, grads, optimizer state, activations: several GB) exceeds the 126 MB L2",
                "step_counter_preset": PRECOND_FREQ - 1,
            },
            "steady_ms_per_step": steady_ms,
            "optimizer_step_ms": optimizer_ms,
            "refresh_step_ms": refresh_ms,
            "first_refresh_step_ms": first_ms,
            "amortized_ms_per_step": amortized(steady_ms),
            "precondition_frequency": PRECOND_FREQ,
            "final_loss": m["final_loss"],
            "clocks": clocks,
            "e2e": {
                "value": e2e_value,
                "unit": "tokens/s",
                "ms_per_step": amortized(e2e_ms),
                "steady_ms_per_step": e2e_ms,
                "h2d_bytes_per_step": m["h2d"],
                "d2h_bytes_per_step": m["d2h"],
            },
            "gpu_launches": launches_per_step * args.steps,
        }
        if other is not None:
            out["other_parallelism"] = {
                "parallelism": describe(other)[0], "comm": describe(other)[1], "value": other["value"], "unit": "tokens/s",
                "amortized_ms_per_step": other["amortized_ms"], "steady_ms_per_step": other["steady_ms"],
                "optimizer_step_ms": other["optimizer_ms"], "refresh_step_ms": other["refresh_ms"],
                "e2e_value": other["e2e_value"],
            }
        if plain is not None:
            out["plain_model"] = {
                "what": "this framework's optimizer under the plain PyTorch GPT-2 of the reference arm (steady steps)",
                "steady_ms_per_step": plain_ms,
                "optimizer_step_ms": plain_opt_ms,
            }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
