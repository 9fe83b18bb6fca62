"""Sharded distributors against the unmodified reference library inside the same gloo ranks:
FSDP1, HSDP1, fully-shard (default assignment) and hybrid-shard (default assignment) must update
the model bit for bit like the reference's distributors do (the reference checks FSDP == HSDP and
per-rank state the same way: ``distributed_shampoo/distributor/gpu_tests/``).  Also the DDP corner
cases of ``shampoo_ddp_distributor_test.py:318-362, 782-858``: ranks without blocks, parameters
without gradients, layers that never receive one."""

import pytest
import torch

from dist_utils_for_tests import run_distributed
from ref_oracle import REF_DIR, reference_available

needs_reference = pytest.mark.skipif(not reference_available(), reason="reference library is not installed under baseline/_ref")


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(
        torch.nn.Linear(12, 20, bias=True), torch.nn.ReLU(), torch.nn.Linear(20, 9, bias=False), torch.nn.ReLU(), torch.nn.Linear(9, 5)
    )


def _data(steps):
    g = torch.Generator().manual_seed(3)
    return [(torch.randn(8, 12, generator=g), torch.randint(0, 5, (8,), generator=g)) for _ in range(steps)]


def _flatten_state(tree, path=""):
    """The state tree of this rank as ``(path, description)`` pairs: for a DTensor its local tensor
    together with the ranks of its mesh and its placements, for a tensor itself, for anything else
    its repr.  Picklable, so that the parent process compares what the ranks saw."""
    from torch.distributed.tensor import DTensor

    out = []
    if isinstance(tree, dict):
        for k in sorted(tree, key=str):
            out += _flatten_state(tree[k], f"{path}/{k}")
    elif isinstance(tree, DTensor):
        out.append((path, ("dtensor", tree.to_local().detach().clone(), tree.device_mesh.mesh.tolist(),
                           [str(p) for p in tree.placements], tuple(tree.shape))))
    elif isinstance(tree, torch.Tensor):
        out.append((path, ("tensor", tree.detach().clone())))
    else:
        out.append((path, ("other", repr(tree))))
    return out


def _assert_same_state(theirs, ours):
    assert [p for p, _ in theirs] == [p for p, _ in ours]
    for (path, a), (_, b) in zip(theirs, ours):
        assert a[0] == b[0], (path, a[0], b[0])
        if a[0] == "other":
            assert a[1] == b[1], path
            continue
        assert a[1].dtype == b[1].dtype and a[1].shape == b[1].shape and torch.equal(a[1], b[1]), path
        assert a[2:] == b[2:], (path, a[2:], b[2:])  # mesh ranks, placements and global shape of a DTensor


def _parity_worker(rank, world, strategy):
    import sys

    sys.path.insert(0, REF_DIR)
    import distributed_shampoo as ref_lib
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, ShardingStrategy, fully_shard
    from torch.distributed.tensor import DTensor

    import optimizers_b200 as our_lib

    def train(lib):
        model = _model()
        cpu = torch.device("cpu")
        if strategy == "ddp":
            model = torch.nn.parallel.DistributedDataParallel(model)
            cfg = lib.DDPDistributedConfig(communication_dtype=torch.float32, num_trainers_per_group=world)
        elif strategy == "fsdp":
            model = FSDP(model, use_orig_params=True, device_id=cpu)
            cfg = lib.FSDPDistributedConfig(param_to_metadata=lib.compile_fsdp_parameter_metadata(model))
        elif strategy == "hsdp":
            mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
            model = FSDP(model, device_mesh=mesh, sharding_strategy=ShardingStrategy.HYBRID_SHARD, use_orig_params=True, device_id=cpu)
            cfg = lib.HSDPDistributedConfig(param_to_metadata=lib.compile_fsdp_parameter_metadata(model), device_mesh=mesh)
        elif strategy == "fully_shard":
            fully_shard(model, mesh=init_device_mesh("cpu", (world,)))
            cfg = lib.FullyShardDistributedConfig()
        else:
            mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
            fully_shard(model, mesh=mesh)
            cfg = lib.HybridShardDistributedConfig(device_mesh=mesh)
        opt = lib.DistributedShampoo(
            model.parameters(), lr=0.01, betas=(0.9, 0.999), epsilon=1e-8, max_preconditioner_dim=8,
            precondition_frequency=2, start_preconditioning_step=2, weight_decay=1e-3,
            grafting_config=lib.AdamPreconditionerConfig(), distributed_config=cfg,
        )
        for x, y in _data(6):
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
        local = [
            (p.to_local() if isinstance(p, DTensor) else p).detach().clone() for p in model.parameters()
        ]
        state_keys = sorted(str(k) for s in opt.state_dict()["state"].values() for k in s)
        return local, state_keys, _flatten_state(opt.state_dict()["state"])

    theirs, their_keys, their_state = train(ref_lib)
    ours, our_keys, our_state = train(our_lib)
    return theirs, ours, their_keys, our_keys, their_state, our_state


@needs_reference
@pytest.mark.parametrize("strategy,world", [("ddp", 2), ("ddp", 3), ("fsdp", 2), ("hsdp", 4), ("fully_shard", 2), ("hybrid_shard", 4)])
def test_sharded_distributor_matches_reference_bitwise(strategy, world):
    """Parameters and, leaf by leaf, the whole per-rank optimizer state (values, block ids, and for
    DTensor state the mesh ranks, placements and global shapes) against the reference's distributor
    run in the same processes (reference: distributor/gpu_tests/shampoo_ddp_distributor_test.py:364-780
    pins the same trees as literals)."""
    for theirs, ours, their_keys, our_keys, their_state, our_state in run_distributed(_parity_worker, world, strategy):
        assert len(theirs) == len(ours)
        for a, b in zip(theirs, ours):
            assert a.shape == b.shape and torch.equal(a, b), (a - b).abs().max()
        assert their_keys == our_keys  # same per-rank block ids and state names
        _assert_same_state(their_state, our_state)


def _ddp_corner_worker(rank, world, case):
    import optimizers_b200 as lib

    torch.manual_seed(0)
    if case == "few_blocks":
        # one parameter, one block: every rank but its owner holds no block at all
        model = torch.nn.Sequential(torch.nn.Linear(6, 4, bias=False))
    else:
        model = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.ReLU(), torch.nn.Linear(8, 4), torch.nn.Linear(4, 3))
    def make(cfg):
        return lib.DistributedShampoo(
            model.parameters(), lr=0.01, betas=(0.9, 0.999), epsilon=1e-8, max_preconditioner_dim=8,
            precondition_frequency=2, start_preconditioning_step=2, grafting_config=lib.AdaGradPreconditionerConfig(epsilon=1e-8),
            distributed_config=cfg,
        )

    opt = make(lib.DDPDistributedConfig(communication_dtype=torch.float32, num_trainers_per_group=world))
    # Creating a mesh is collective.  Every rank, also one that owns no block and therefore never
    # allocates state, must have created the owners' mesh by now (gloo tolerates a subset of ranks
    # creating it later; NCCL with communicators bound at start-up hangs).
    from optimizers_b200.parallel.dist_utils import get_device_mesh

    assert get_device_mesh.cache_info().currsize >= 1
    g = torch.Generator().manual_seed(5)
    for step in range(5):
        x = torch.randn(8, 6, generator=g)
        opt.zero_grad(set_to_none=True)
        if case == "dead_layer":
            out = model[1](model[0](x))
            out = model[2](out)  # the last layer never takes part: its gradients stay None
        else:
            out = model(x)
        out.square().mean().backward()
        if case == "missing_grads" and step % 2 == 1:
            # gradients vanish on some steps (same on every rank), as under gradient accumulation masks
            list(model.parameters())[0].grad = None
        opt.step()
    return [p.detach().clone() for p in model.parameters()]


def _single_corner(case):
    """The same training loop on one process with the single-device distributor."""
    import optimizers_b200 as lib

    class _Stub:
        pass

    torch.manual_seed(0)
    if case == "few_blocks":
        model = torch.nn.Sequential(torch.nn.Linear(6, 4, bias=False))
    else:
        model = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.ReLU(), torch.nn.Linear(8, 4), torch.nn.Linear(4, 3))
    opt = lib.DistributedShampoo(
        model.parameters(), lr=0.01, betas=(0.9, 0.999), epsilon=1e-8, max_preconditioner_dim=8,
        precondition_frequency=2, start_preconditioning_step=2, grafting_config=lib.AdaGradPreconditionerConfig(epsilon=1e-8),
    )
    g = torch.Generator().manual_seed(5)
    for step in range(5):
        x = torch.randn(8, 6, generator=g)
        opt.zero_grad(set_to_none=True)
        if case == "dead_layer":
            out = model[2](model[1](model[0](x)))
        else:
            out = model(x)
        out.square().mean().backward()
        if case == "missing_grads" and step % 2 == 1:
            list(model.parameters())[0].grad = None
        opt.step()
    return [p.detach().clone() for p in model.parameters()]


@pytest.mark.parametrize("case,world", [("few_blocks", 3), ("missing_grads", 2), ("dead_layer", 2)])
def test_ddp_ranks_without_blocks_and_parameters_without_gradients(case, world):
    ref = _single_corner(case)
    for params in run_distributed(_ddp_corner_worker, world, case):
        for a, b in zip(ref, params):
            assert torch.equal(a, b), (a - b).abs().max()


def _random_options_worker(rank, world, strategy, seeds):
    """For every seed: one random option set (see test_random_option_sets_parity) and random
    distributor options, trained under ``strategy`` by the reference and by this library in the
    same ranks; returns, per seed, both outcomes and whether the local parameters are identical."""
    import logging
    import math
    import random
    import sys

    sys.path.insert(0, REF_DIR)
    import distributed_shampoo as ref_lib
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, ShardingStrategy, fully_shard
    from torch.distributed.tensor import DTensor

    import optimizers_b200 as our_lib
    import test_random_option_sets_parity as option_sets

    logging.disable(logging.WARNING)
    results = []
    for seed in seeds:

        def train(lib):
            rng = random.Random(seed)
            family, kw = option_sets._options(lib, rng)
            if family == "spectral":  # needs whole matrices: not a distributor topic
                return "skipped", None
            if kw["max_preconditioner_dim"] == math.inf:
                kw["max_preconditioner_dim"] = 8
            torch.manual_seed(seed)
            model = _model()
            cpu = torch.device("cpu")
            comm_dtype = rng.choice([torch.float32, torch.bfloat16])
            if strategy == "ddp":
                model = torch.nn.parallel.DistributedDataParallel(model)
                cfg = lib.DDPDistributedConfig(
                    communication_dtype=comm_dtype, num_trainers_per_group=rng.choice([-1, world]),
                    communicate_params=rng.random() < 0.5,
                )
            elif strategy == "hsdp":
                mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
                model = FSDP(model, device_mesh=mesh, sharding_strategy=ShardingStrategy.HYBRID_SHARD, use_orig_params=True, device_id=cpu)
                cfg = lib.HSDPDistributedConfig(
                    param_to_metadata=lib.compile_fsdp_parameter_metadata(model), device_mesh=mesh,
                    communication_dtype=comm_dtype, communicate_params=rng.random() < 0.5,
                )
            elif strategy == "fully_shard_replicate":
                fully_shard(model, mesh=init_device_mesh("cpu", (world,)))
                cfg = lib.FullyShardDistributedConfig(
                    param_assignment_strategy=lib.FSDPParamAssignmentStrategy.REPLICATE, num_sub_groups=rng.choice([1, 2])
                )
            else:
                mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
                fully_shard(model, mesh=mesh)
                cfg = lib.HybridShardDistributedConfig(device_mesh=mesh, communication_dtype=comm_dtype)
            kw["distributed_config"] = cfg
            try:
                opt = lib.DistributedShampoo(model.parameters(), **kw)
            except Exception as err:  # noqa: BLE001 - the kind and the text are what is compared
                return f"constructor: {type(err).__name__}: {option_sets._strip(str(err))}", None
            g = torch.Generator().manual_seed(seed + 1 + rank)
            opt.train()
            try:
                for step in range(6):
                    x, y = torch.randn(8, 12, generator=g), torch.randint(0, 5, (8,), generator=g)
                    opt.zero_grad()
                    torch.nn.functional.cross_entropy(model(x), y).backward()
                    opt.step()
                    if step == 3:
                        opt.eval()
                        opt.train()
                opt.eval()
            except Exception as err:  # noqa: BLE001
                return f"step: {type(err).__name__}: {option_sets._strip(str(err))}", None
            return "trained", [(p.to_local() if isinstance(p, DTensor) else p).detach().clone() for p in model.parameters()]

        theirs, their_params = train(ref_lib)
        dist.barrier()
        mine, my_params = train(our_lib)
        dist.barrier()
        identical = their_params is None or all(
            a.shape == b.shape and torch.equal(a, b) for a, b in zip(their_params, my_params, strict=True)
        )
        results.append((seed, theirs, mine, identical))
    return results


@needs_reference
@pytest.mark.parametrize("strategy,world", [("ddp", 2), ("hsdp", 4), ("fully_shard_replicate", 2), ("hybrid_shard", 4)])
def test_random_option_sets_under_distributors_match_reference_bitwise(strategy, world):
    """Eight random option sets per strategy (with random communication dtype, parameter or
    direction communication, group size, sub-groups): every rank ends with the reference's local
    parameters, bit for bit, including a visit to eval mode."""
    per_rank = run_distributed(_random_options_worker, world, strategy, list(range(8)))
    trained = 0
    for results in per_rank:
        for seed, theirs, mine, identical in results:
            assert theirs == mine, (strategy, seed, theirs, mine)
            assert identical, (strategy, seed)
            trained += theirs == "trained"
    assert trained >= 5 * world
