"""Worker for the multi-GPU tests: trains a small MLP with the native DDP engine and writes the
final parameters of rank 0.  Launched by test_gpu_multi.py through torch.distributed.run."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    mode, out = sys.argv[1], sys.argv[2]
    bf16_comm = mode.endswith("+bf16")  # search directions travel in bf16, as in the benchmarks
    mode = mode.removesuffix("+bf16")
    comm_params = mode.endswith("+params")  # updated parameters travel instead of search directions
    mode = mode.removesuffix("+params")
    dead = mode.endswith("+dead")  # a registered layer that the forward pass never uses: its gradient stays None
    mode = mode.removesuffix("+dead")
    tiny = mode.endswith("+tiny")  # a single block: every rank but one owns nothing
    mode = mode.removesuffix("+tiny")
    from optimizers_b200 import (
        AdamPreconditionerConfig,
        DDPDistributedConfig,
        DistributedShampoo,
        NativeRuntimeConfig,
    )

    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    features = 16 if tiny else 96

    class Net(torch.nn.Module):
        def __init__(self) -> None:
            super().__init__()
            if tiny:
                self.body = torch.nn.Sequential(torch.nn.Linear(features, 10, bias=False))
            else:
                self.body = torch.nn.Sequential(
                    torch.nn.Linear(96, 200), torch.nn.ReLU(), torch.nn.Linear(200, 72), torch.nn.ReLU(), torch.nn.Linear(72, 10)
                )
            if dead:
                self.unused = torch.nn.Linear(24, 40)

        def forward(self, x):
            return self.body(x)

    model = Net().to(dev)
    fused = mode == "p2p_pull"
    train_model = model if fused else torch.nn.parallel.DistributedDataParallel(
        model, device_ids=[dev.index], find_unused_parameters=dead
    )
    native = NativeRuntimeConfig(
        backend="torch" if mode == "torch" else "native",
        comm_path="p2p" if mode.startswith("p2p") else "nccl",
        fuse_gradient_reduction=fused,
        fuse_direction_push=mode == "p2p_gemm",
    )
    opt = DistributedShampoo(
        model.parameters(), lr=1e-3, betas=(0.9, 0.999), epsilon=1e-6, max_preconditioner_dim=64,
        precondition_frequency=3, start_preconditioning_step=3, weight_decay=1e-2,
        grafting_config=AdamPreconditionerConfig(),
        distributed_config=DDPDistributedConfig(
            communication_dtype=torch.bfloat16 if bf16_comm else torch.float32, num_trainers_per_group=world,
            communicate_params=comm_params,
        ),
        native_runtime_config=native,
    )
    g = torch.Generator(device="cuda").manual_seed(1)
    for _ in range(8):
        x = torch.randn(64, 96, device=dev, generator=g)[:, :features]
        y = torch.randint(0, 10, (64,), device=dev, generator=g)
        shard = slice(rank * 64 // world, (rank + 1) * 64 // world)
        opt.zero_grad(set_to_none=not fused)
        torch.nn.functional.cross_entropy(train_model(x[shard]), y[shard]).backward()
        opt.step()
    for rec in opt._per_group_state_lists:
        if rec.get("native_engine") is not None:
            rec["native_engine"].check_status()
            arena = getattr(rec["native_engine"], "_arena", None)
            assert arena is None or arena.overrun_regions() == [], arena.overrun_regions()
            pushed = rec["native_engine"].gemm_push_steps
            # 8 steps, preconditioning from step 3: six steps gather from the GEMM epilogue
            assert pushed == (6 if mode == "p2p_gemm" else 0), pushed
        else:
            assert mode == "torch"
    torch.cuda.synchronize()
    params = [p.detach().cpu() for p in model.parameters()]
    gathered = [None] * world
    dist.all_gather_object(gathered, params)
    if rank == 0:
        for other in gathered[1:]:
            for a, b in zip(gathered[0], other):
                assert torch.equal(a, b), "ranks diverged"
        torch.save(params, out)
    dist.destroy_process_group()


def sharded_main() -> None:
    """``<backend>:<strategy>``: train the MLP under one of the sharded strategies with the torch
    or the native step and write rank 0's view of the full final parameters."""
    mode, out = sys.argv[1], sys.argv[2]
    backend, strategy, *rest = mode.split(":")
    comm_path = "p2p" if "p2p" in rest else "nccl"
    gpa = "gpa" in rest  # primal averaging: the saved parameters are those of eval mode
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, fully_shard, ShardingStrategy
    from torch.distributed.tensor import DTensor

    from optimizers_b200 import (
        AdaGradPreconditionerConfig,
        compile_fsdp_parameter_metadata,
        DistributedShampoo,
        FSDPDistributedConfig,
        FSDPParamAssignmentStrategy,
        FullyShardDistributedConfig,
        HSDPDistributedConfig,
        HybridShardDistributedConfig,
        GeneralizedPrimalAveragingConfig,
        NativeRuntimeConfig,
    )

    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    model = torch.nn.Sequential(
        torch.nn.Linear(96, 200, bias=False), torch.nn.ReLU(), torch.nn.Linear(200, 72, bias=False), torch.nn.ReLU(),
        torch.nn.Linear(72, 10, bias=False),
    ).to(dev)
    # FSDP1's hybrid strategy needs a shard dimension of at least 2 to flatten its parameters.
    mesh_shape = (world // 2, 2) if strategy == "hsdp" else (2, world // 2)
    mesh2d = init_device_mesh("cuda", mesh_shape, mesh_dim_names=("replicate", "shard")) if "h" == strategy[0] else None
    lossless = {
        "fully_shard_rr": FSDPParamAssignmentStrategy.ROUND_ROBIN,
        "fully_shard_rep": FSDPParamAssignmentStrategy.REPLICATE,
        "hybrid_shard_rr": FSDPParamAssignmentStrategy.ROUND_ROBIN,
    }
    if strategy == "fsdp":
        model = FSDP(model, use_orig_params=True)
        dc = FSDPDistributedConfig(param_to_metadata=compile_fsdp_parameter_metadata(model))
    elif strategy == "hsdp":
        model = FSDP(model, device_mesh=mesh2d, sharding_strategy=ShardingStrategy.HYBRID_SHARD, use_orig_params=True)
        dc = HSDPDistributedConfig(param_to_metadata=compile_fsdp_parameter_metadata(model), device_mesh=mesh2d)
    elif strategy.startswith("fully_shard"):
        model = fully_shard(model)
        dc = FullyShardDistributedConfig(
            param_assignment_strategy=lossless.get(strategy, FSDPParamAssignmentStrategy.DEFAULT)
        )
    else:
        model = fully_shard(model, mesh=mesh2d)
        dc = HybridShardDistributedConfig(
            device_mesh=mesh2d, param_assignment_strategy=lossless.get(strategy, FSDPParamAssignmentStrategy.DEFAULT)
        )
    opt = DistributedShampoo(
        model.parameters(), lr=1e-3, betas=(0.9, 0.999), epsilon=1e-6, max_preconditioner_dim=64,
        precondition_frequency=3, start_preconditioning_step=3, weight_decay=1e-2,
        grafting_config=AdaGradPreconditionerConfig(epsilon=1e-8), distributed_config=dc,
        native_runtime_config=NativeRuntimeConfig(backend=backend, comm_path=comm_path),
        **({"iterate_averaging_config": GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.9, train_interp_coeff=0.7)} if gpa else {}),
    )
    if gpa:
        opt.train()
    g = torch.Generator(device="cuda").manual_seed(1)
    for _ in range(8):
        x = torch.randn(64, 96, device=dev, generator=g)
        y = torch.randint(0, 10, (64,), device=dev, generator=g)
        shard = slice(rank * 64 // world, (rank + 1) * 64 // world)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x[shard]), y[shard]).backward()
        opt.step()
    if gpa:
        opt.eval()  # what an evaluation or a checkpoint would see: the averaged x sequence
    if comm_path == "p2p":
        for rec in opt._per_group_state_lists:
            d = rec["distributor"]
            if getattr(d, "_gather_grads_ctx", None) is None:
                # DDP-family distributor: the engine stores the directions into the peers' buffers
                assert rec["native_engine"] is None or rec["native_engine"]._p2p
                continue
            if d._gather_grads_ctx._group_size > 1:  # a shard group of one rank has nothing to exchange
                assert d._gather_grads_ctx._p2p and d._redistribute_ctx._p2p
            d._gather_grads_ctx.check_status()
            d._redistribute_ctx.check_status()
            for ctx in (d._gather_grads_ctx, d._redistribute_ctx):
                arena = getattr(ctx, "_arena", None)
                assert arena is None or arena.overrun_regions() == [], arena.overrun_regions()
    engines = [rec.get("native_engine") for rec in opt._per_group_state_lists]
    assert all((e is not None) == (backend == "native") for e in engines), engines
    for e in engines:
        if e is not None:
            e.check_status()
            arena = getattr(e, "_arena", None)
            assert arena is None or arena.overrun_regions() == [], arena.overrun_regions()
    torch.cuda.synchronize()
    if strategy in ("fsdp", "hsdp"):
        with FSDP.summon_full_params(model):
            params = [p.detach().cpu().clone() for p in model.parameters()]
    else:
        params = [p.full_tensor().cpu() if isinstance(p, DTensor) else p.detach().cpu() for p in model.parameters()]
    if rank == 0:
        torch.save(params, out)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    sharded_main() if ":" in sys.argv[1] else main()
