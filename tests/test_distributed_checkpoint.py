"""Distributed checkpointing (torch.distributed.checkpoint) of the sharded optimizers on gloo
ranks: training interrupted by a save, a fresh model + optimizer and a load continues bit for bit
like training that was never interrupted (the reference's pre-emption test,
``distributed_shampoo/distributor/gpu_tests/shampoo_checkpoint_test.py:317-485``)."""

import pytest
import torch

from dist_utils_for_tests import run_distributed

INITIAL, CONTINUED = 5, 5


def _build(rank, world, hybrid, strategy_name):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import optimizers_b200 as lib

    torch.manual_seed(0)
    model = torch.nn.Sequential(
        torch.nn.Linear(12, 20, bias=False), torch.nn.ReLU(), torch.nn.Linear(20, 9, bias=False), torch.nn.ReLU(),
        torch.nn.Linear(9, 5, bias=False),
    )
    strategy = lib.FSDPParamAssignmentStrategy[strategy_name]
    if hybrid:
        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
        fully_shard(model, mesh=mesh)
        cfg = lib.HybridShardDistributedConfig(device_mesh=mesh, param_assignment_strategy=strategy)
    else:
        fully_shard(model, mesh=init_device_mesh("cpu", (world,)))
        cfg = lib.FullyShardDistributedConfig(param_assignment_strategy=strategy)
    opt = lib.DistributedShampoo(
        model.parameters(), lr=0.01, betas=(0.9, 0.999), epsilon=1e-8, max_preconditioner_dim=8,
        precondition_frequency=2, start_preconditioning_step=2, weight_decay=1e-3,
        grafting_config=lib.AdaGradPreconditionerConfig(epsilon=1e-8), distributed_config=cfg,
    )
    return model, opt


def _step(model, opt, x):
    loss = model(x).square().sum()
    loss.backward()
    opt.step()
    opt.zero_grad()
    return loss.detach().clone()


def _flat_state(opt):
    from torch.distributed.tensor import DTensor

    out = {}

    def walk(prefix, obj):
        if isinstance(obj, dict):
            for k, v in obj.items():
                walk(f"{prefix}/{k}", v)
        elif isinstance(obj, torch.Tensor):
            out[prefix] = (obj.to_local() if isinstance(obj, DTensor) else obj).detach().clone()

    walk("", opt.state_dict()["state"])
    return out


def _preemption_worker(rank, world, hybrid, strategy_name, directory):
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.state_dict import get_model_state_dict, get_optimizer_state_dict, set_model_state_dict, set_optimizer_state_dict

    model1, opt1 = _build(rank, world, hybrid, strategy_name)
    g = torch.Generator().manual_seed(42 + rank)  # every rank trains on its own data
    data = [torch.randn(4, 12, generator=g) for _ in range(INITIAL + CONTINUED)]
    for x in data[:INITIAL]:
        _step(model1, opt1, x)
    dcp.save(
        {"model": get_model_state_dict(model1), "optimizer": get_optimizer_state_dict(model1, opt1)},
        storage_writer=dcp.FileSystemWriter(directory),
    )
    losses1 = [_step(model1, opt1, x) for x in data[INITIAL:]]

    # the job is pre-empted and restarted: new objects, different initial weights, then the load
    model2, opt2 = _build(rank, world, hybrid, strategy_name)
    with torch.no_grad():
        for p in model2.parameters():
            p.add_(1.0)
    state = {"model": get_model_state_dict(model2), "optimizer": get_optimizer_state_dict(model2, opt2)}
    dcp.load(state, storage_reader=dcp.FileSystemReader(directory))
    set_model_state_dict(model2, state["model"])
    set_optimizer_state_dict(model2, opt2, state["optimizer"])
    losses2 = [_step(model2, opt2, x) for x in data[INITIAL:]]
    dist.barrier()
    s1, s2 = _flat_state(opt1), _flat_state(opt2)
    params = [(a.to_local().clone(), b.to_local().clone()) for a, b in zip(model1.parameters(), model2.parameters())]
    return losses1, losses2, s1, s2, params


@pytest.mark.parametrize("hybrid,world", [(False, 2), (True, 4)])
@pytest.mark.parametrize("strategy", ["REPLICATE", "ROUND_ROBIN", "DEFAULT"])
def test_preemption_resumes_bitwise(tmp_path, hybrid, world, strategy):
    for losses1, losses2, s1, s2, params in run_distributed(_preemption_worker, world, hybrid, strategy, str(tmp_path / "ckpt")):
        for a, b in zip(losses1, losses2):
            assert torch.equal(a, b)
        assert s1.keys() == s2.keys() and len(s1) > 0
        for k in s1:
            assert torch.equal(s1[k], s2[k]), k
        for a, b in params:
            assert torch.equal(a, b)
