"""Training throughput of the two other model configurations the optimizer is specified on:

  resnet18   ResNet-18 (CIFAR variant), batch 128 per GPU of 3x32x32 N(0,1) images, Shampoo with
             max_preconditioner_dim=1024, precondition_frequency=50, Adam grafting, momentum 0.9;
             N > 1: torch DDP + the DDP distributor with a bf16 search-direction all-gather
  llama1b    Llama-style 1B decoder (16 layers, d_model 2048, 32 heads, SwiGLU 8192, vocab 32000),
             batch 4 x 2048 tokens per GPU, bf16 autocast, eigenvalue-corrected Shampoo (SOAP) with
             QR-iteration eigenbasis refresh every 50 steps, max_preconditioner_dim=4096;
             N > 1: fully_shard (FSDP2) + the fully-shard distributor

Same protocol as ``bench.py``: synthetic data resident on the device, W warm-up steps, K steps timed
with CUDA events between barriers, maximum over ranks, one JSON line from rank 0.  ``--impl
reference`` runs the unmodified reference optimizer from ``baseline/_ref`` under the same (plain
PyTorch, ``fused=False``) model definition.

    python benchmarks/train_throughput.py --config resnet18 --steps 20
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/train_throughput.py --config resnet18
    python benchmarks/train_throughput.py --config llama1b --steps 5 --warmup 3
"""

from __future__ import annotations

import argparse
import json
import os
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", choices=["resnet18", "llama1b"], default="resnet18")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--backend", default="auto", help="native runtime back-end of this framework")
    ap.add_argument("--comm", choices=["nccl", "p2p"], default="p2p",
                    help="N > 1, this framework: gather the search directions with NCCL or by peer stores (DDP family)")
    ap.add_argument("--layers", type=int, default=None, help="debug: fewer decoder layers")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
        import distributed_shampoo as lib

        extra = {}
    else:
        import optimizers_b200 as lib

        extra = {"native_runtime_config": lib.NativeRuntimeConfig(backend=args.backend, comm_path=args.comm if world > 1 else "nccl")}
    from optimizers_b200 import models as M

    if not hasattr(lib, "ClassicMomentumConfig"):  # the reference defines it but does not re-export it
        from distributed_shampoo.shampoo_types import ClassicMomentumConfig

        lib.ClassicMomentumConfig = ClassicMomentumConfig

    torch.manual_seed(1234)
    torch.backends.cuda.matmul.allow_tf32 = False
    fused = args.impl == "ours"
    if args.config == "resnet18":
        model = M.ResNet18().to(dev)
        train_model = model
        dist_cfg = lib.DefaultSingleDeviceDistributedConfig
        if world > 1:
            train_model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank])
            dist_cfg = lib.DDPDistributedConfig(communication_dtype=torch.bfloat16, num_trainers_per_group=world)
        opt = lib.DistributedShampoo(
            model.parameters(), lr=1e-3, betas=(0.9, 0.999), epsilon=1e-12, max_preconditioner_dim=1024,
            precondition_frequency=50, start_preconditioning_step=50,
            grafting_config=lib.AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8),
            iterate_averaging_config=lib.ClassicMomentumConfig(momentum=0.9),
            distributed_config=dist_cfg, **extra,
        )
        period, per_gpu, unit = 50, 128, "images/s"
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        data = [
            (torch.randn(per_gpu, 3, 32, 32, device=dev, generator=g), torch.randint(0, 10, (per_gpu,), device=dev, generator=g))
            for _ in range(4)
        ]

        def step(i: int):
            x, y = data[i % 4]
            loss = torch.nn.functional.cross_entropy(train_model(x), y)
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            return loss
    else:
        cfg = M.LlamaConfig(fused=fused) if args.layers is None else M.LlamaConfig(fused=fused, n_layer=args.layers)
        model = M.Llama(cfg).to(dev)
        dist_cfg = lib.DefaultSingleDeviceDistributedConfig
        if world > 1:
            from torch.distributed.fsdp import fully_shard

            for layer in model.layers:
                fully_shard(layer)
            fully_shard(model)
            dist_cfg = lib.FullyShardDistributedConfig()
        opt = lib.DistributedShampoo(
            model.parameters(), lr=3e-4, betas=(0.9, 0.999), epsilon=1e-12, max_preconditioner_dim=4096,
            precondition_frequency=50, start_preconditioning_step=50,
            preconditioner_config=lib.EigenvalueCorrectedShampooPreconditionerConfig(
                amortized_computation_config=lib.QREigendecompositionConfig()
            ),
            grafting_config=None, distributed_config=dist_cfg, **extra,
        )
        period, seq = 50, 2048
        per_gpu, unit = 4 * seq, "tokens/s"
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        data = [torch.randint(0, cfg.vocab_size, (4, seq + 1), device=dev, generator=g) for _ in range(4)]

        def step(i: int):
            t = data[i % 4]
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = model(t[:, :-1], t[:, 1:])
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            return loss

    # Resume-style preset of the shared step counter: the first warm-up step is the first
    # preconditioned one (and performs the amortised computation).
    for state in opt.state.values():
        if "step" in state:
            state["step"].fill_(period - 1)
            break

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 1)):
        step(i)
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        loss = step(i)
    stop.record()
    barrier()
    ms = torch.tensor([start.elapsed_time(stop)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    native = None
    if args.impl == "ours":
        native = all(rec.get("native_engine") is not None for rec in opt._per_group_state_lists)
    if rank == 0:
        print(json.dumps({
            "config": args.config, "impl": args.impl, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "value": per_gpu * world * args.steps / (ms_total / 1e3), "unit": unit,
            "native_engine": native, "final_loss": float(loss.item()),
            "peak_memory_gb": round(torch.cuda.max_memory_allocated(dev) / 2**30, 2),
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
