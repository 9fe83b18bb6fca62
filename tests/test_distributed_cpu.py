"""Multi-process CPU (gloo) tests of the distributors: the distributed optimizers must agree with
single-device Shampoo (bitwise for fp32 communication)."""

import copy

import pytest
import torch

from dist_utils_for_tests import run_distributed


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(
        torch.nn.Linear(12, 20, bias=True), torch.nn.ReLU(), torch.nn.Linear(20, 9, bias=False), torch.nn.ReLU(), torch.nn.Linear(9, 5)
    )


def _opt_kwargs():
    from optimizers_b200 import AdamPreconditionerConfig

    return dict(
        lr=0.01, betas=(0.9, 0.999), epsilon=1e-8, max_preconditioner_dim=8, precondition_frequency=2,
        start_preconditioning_step=2, weight_decay=1e-3, grafting_config=AdamPreconditionerConfig(),
    )


def _data(steps):
    g = torch.Generator().manual_seed(3)
    return [(torch.randn(8, 12, generator=g), torch.randint(0, 5, (8,), generator=g)) for _ in range(steps)]


def _train_single(steps=5):
    from optimizers_b200 import DistributedShampoo

    model = _model()
    opt = DistributedShampoo(model.parameters(), **_opt_kwargs())
    for x, y in _data(steps):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    return [p.detach().clone() for p in model.parameters()]


def _ddp_worker(rank, world, comm_dtype_name, group_size):
    import torch.distributed as dist

    from optimizers_b200 import DDPDistributedConfig, DistributedShampoo

    model = _model()
    cfg = DDPDistributedConfig(communication_dtype=getattr(torch, comm_dtype_name), num_trainers_per_group=group_size)
    opt = DistributedShampoo(model.parameters(), distributed_config=cfg, **_opt_kwargs())
    for x, y in _data(5):
        opt.zero_grad()
        # every rank sees the full batch, so gradients equal the single-device ones
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    state = opt.state_dict()["state"]
    n_blocks = sum(1 for s in state.values() for k in s if str(k).startswith("block_"))
    return [p.detach().clone() for p in model.parameters()], n_blocks


@pytest.mark.parametrize("world,group", [(2, 2), (4, 2), (3, -1)])
def test_ddp_fp32_matches_single_device_bitwise(world, group):
    ref = _train_single()
    results = run_distributed(_ddp_worker, world, "float32", group)
    for params, _ in results:
        for a, b in zip(ref, params):
            assert torch.equal(a, b)
    # every block is owned by exactly one rank of each group
    n_groups = 1 if group == -1 else world // group
    assert sum(n for _, n in results) % n_groups == 0


def test_ddp_bf16_close_to_single_device():
    ref = _train_single()
    for params, _ in run_distributed(_ddp_worker, 2, "bfloat16", 2):
        for a, b in zip(ref, params):
            assert torch.allclose(a, b, rtol=2e-2, atol=2e-3)


def _fully_shard_worker(rank, world, strategy_name, num_sub_groups, mesh_shape):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    from optimizers_b200 import (
        DistributedShampoo,
        FSDPParamAssignmentStrategy,
        FullyShardDistributedConfig,
        HybridShardDistributedConfig,
    )

    model = _model()
    strategy = FSDPParamAssignmentStrategy[strategy_name]
    if mesh_shape is None:
        mesh = init_device_mesh("cpu", (world,))
        cfg = FullyShardDistributedConfig(param_assignment_strategy=strategy, num_sub_groups=num_sub_groups)
    else:
        mesh = init_device_mesh("cpu", mesh_shape, mesh_dim_names=("replicate", "shard"))
        cfg = HybridShardDistributedConfig(
            param_assignment_strategy=strategy, num_sub_groups=num_sub_groups, device_mesh=mesh
        )
    fully_shard(model, mesh=mesh)
    opt = DistributedShampoo(model.parameters(), distributed_config=cfg, **_opt_kwargs())
    for x, y in _data(5):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    full = [p.full_tensor().detach().clone() for p in model.parameters()]
    keys = sorted({str(k) for s in opt.state_dict()["state"].values() for k in s})
    # checkpoint round trip in place
    sd = copy.deepcopy(opt.state_dict())
    opt.load_state_dict(sd)
    return full, keys


@pytest.mark.parametrize("strategy,subgroups", [("ROUND_ROBIN", 1), ("REPLICATE", 1), ("ROUND_ROBIN", 2)])
def test_fully_shard_lossless_matches_single_device(strategy, subgroups):
    ref = _train_single()
    for full, _ in run_distributed(_fully_shard_worker, 2, strategy, subgroups, None):
        for a, b in zip(ref, full):
            assert torch.allclose(a, b, rtol=0, atol=0), (a - b).abs().max()


def test_fully_shard_default_runs_and_uses_rank_block_ids():
    results = run_distributed(_fully_shard_worker, 2, "DEFAULT", 1, None)
    for rank, (full, keys) in enumerate(results):
        assert all(torch.isfinite(t).all() for t in full)
        assert any(k.startswith(f"rank_{rank}-block_") for k in keys)
    for a, b in zip(results[0][0], results[1][0]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("strategy", ["ROUND_ROBIN", "REPLICATE"])
def test_hybrid_shard_lossless_matches_single_device(strategy):
    ref = _train_single()
    for full, _ in run_distributed(_fully_shard_worker, 4, strategy, 1, (2, 2)):
        for a, b in zip(ref, full):
            assert torch.equal(a, b)


def _gpa_idle_rank_worker(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import optimizers_b200 as lib

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(12, 20, bias=False), torch.nn.ReLU(), torch.nn.Linear(20, 9, bias=False))
    if world > 1:
        fully_shard(model, mesh=init_device_mesh("cpu", (world,)))
        extra = {"distributed_config": lib.FullyShardDistributedConfig(param_assignment_strategy=lib.FSDPParamAssignmentStrategy.ROUND_ROBIN)}
    else:
        extra = {}
    opt = lib.DistributedShampoo(
        model.parameters(), lr=0.01, max_preconditioner_dim=8, precondition_frequency=2, start_preconditioning_step=2,
        grafting_config=lib.AdaGradPreconditionerConfig(epsilon=1e-8),
        iterate_averaging_config=lib.GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.9, train_interp_coeff=0.7), **extra,
    )
    opt.train()
    g = torch.Generator().manual_seed(1)
    for _ in range(4):
        x = torch.randn(8, 12, generator=g)
        opt.zero_grad()
        model(x).square().sum().backward()
        opt.step()
    opt.eval()  # a rank that owns no parameter still takes part in the switch's collective
    return [(p.full_tensor() if world > 1 else p).detach().clone() for p in model.parameters()]


def test_primal_averaging_mode_switch_with_a_rank_that_owns_nothing():
    """Two parameters, four ranks, ROUND_ROBIN ownership: two ranks hold no block; train()/eval()
    and the steps must neither fail on them nor change the result (four ranks: the gradient
    average of identical shards is exact)."""
    ref = _gpa_idle_rank_worker(0, 1)
    for params in run_distributed(_gpa_idle_rank_worker, 4):
        for a, b in zip(ref, params):
            assert torch.equal(a, b), (a - b).abs().max()
