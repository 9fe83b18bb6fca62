"""The native engine's orchestration on the CPU.

``tests/fake_block_ext.py`` performs the engine's kernels with torch; the device-only pieces the
engine touches besides (CUDA events, pinned memory, the capability check, the current stream) are
replaced by inert stand-ins.  The engine then steps a model on the CPU and must agree with the
torch step of the same optimizer: plans, tables, selectors, refresh and mirrors, weight decay,
momentum, primal averaging and mode switches, dims switched off, gradients that go missing.
"""

import pytest
import torch

import optimizers_b200 as ob
from fake_block_ext import FakeBlockExt


class _Event:
    def __init__(self, *args, **kwargs):
        pass

    def record(self, *args):
        pass

    def synchronize(self):
        pass

    def query(self):
        return True

    def wait(self, *args):
        pass


class _Stream(_Event):
    def wait_event(self, *args):
        pass

    def wait_stream(self, *args):
        pass


def install_cpu_engine(setattr_):
    """Make ``backend="native"`` build the engine for CPU parameters on top of the stand-in.
    ``setattr_(object, name, value)`` does the patching (pytest's monkeypatch, or plain ``setattr``
    inside a spawned rank)."""
    import optimizers_b200.native_engine as engine_module
    from optimizers_b200.ops import build

    ext = FakeBlockExt()
    setattr_(build, "load", lambda: ext)
    setattr_(build, "available", lambda: True)
    setattr_(
        engine_module, "maybe_build_native_engine",
        lambda optimizer, rec, group, cfg: None if cfg.backend == "torch" else engine_module.build_native_engine(optimizer, rec, group, cfg),
    )
    setattr_(torch.cuda, "Event", _Event)
    setattr_(torch.cuda, "get_device_capability", lambda device=None: (10, 0))
    setattr_(torch.cuda, "current_stream", lambda device=None: _Stream())
    setattr_(torch.Tensor, "pin_memory", lambda self, *args, **kwargs: self)
    return ext


@pytest.fixture
def cpu_engine(monkeypatch):
    return install_cpu_engine(monkeypatch.setattr)


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(20, 36), torch.nn.Tanh(), torch.nn.Linear(36, 12), torch.nn.Tanh(), torch.nn.Linear(12, 4))


def _train(backend, steps=8, visit_eval_at=(), drop_grad_at=(), **kw):
    # epsilon 1e-4: with a ridge of 1e-8 the inverse roots of these rank-deficient factors amplify the
    # difference between two eigensolvers to 1e-4 in the parameters, which would hide a wrong plan
    model = _model()
    args = dict(lr=1e-2, betas=(0.9, 0.999), epsilon=1e-4, max_preconditioner_dim=16, precondition_frequency=3, start_preconditioning_step=3)
    args.update(kw)
    runtime = ob.NativeRuntimeConfig(backend=backend, gemm_mode=args.pop("gemm_mode", "tf32x3"))
    opt = ob.DistributedShampoo(model.parameters(), native_runtime_config=runtime, **args)
    opt.train()
    g = torch.Generator().manual_seed(1)
    seen = []
    for step in range(steps):
        if step in visit_eval_at:
            opt.eval()
            seen.append([p.detach().clone() for p in model.parameters()])
            opt.train()
        x, y = torch.randn(32, 20, generator=g), torch.randint(0, 4, (32,), generator=g)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        if step in drop_grad_at:
            list(model.parameters())[2].grad = None
        opt.step()
    seen.append([p.detach().clone() for p in model.parameters()])
    return seen, opt


def _configs():
    return {
        "adam_graft_weight_decay": dict(grafting_config=ob.AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8), weight_decay=1e-2),
        "no_grafting_unpacked": dict(preconditioner_config=ob.RootInvShampooPreconditionerConfig(use_symmetric_packing=False), beta3=0.8),
        "sgd_graft_l2_nesterov": dict(
            grafting_config=ob.SGDPreconditionerConfig(), weight_decay=1e-3, weight_decay_type=ob.WeightDecayType.L2,
            iterate_averaging_config=ob.ClassicMomentumConfig(momentum=0.5, dampening=0.1, use_nesterov=True),
        ),
        "primal_averaging": dict(
            grafting_config=ob.AdamPreconditionerConfig(), weight_decay=1e-2,
            iterate_averaging_config=ob.GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.9, train_interp_coeff=0.7),
        ),
        "eigendecomposed": dict(grafting_config=ob.AdaGradPreconditionerConfig(), preconditioner_config=ob.EigendecomposedShampooPreconditionerConfig()),
        "kl_root_inverse": dict(grafting_config=ob.AdamPreconditionerConfig(), preconditioner_config=ob.RootInvKLShampooPreconditionerConfig()),
        "kl_eigendecomposed": dict(preconditioner_config=ob.EigendecomposedKLShampooPreconditionerConfig()),
        "single_pass_gemm_mode": dict(grafting_config=ob.AdamPreconditionerConfig(), gemm_mode="tf32"),
        "rmsprop_graft_no_bias_correction": dict(grafting_config=ob.RMSpropPreconditionerConfig(beta2=0.95), use_bias_correction=False),
        # Eigenvectors inside a (nearly) multiple eigenvalue are arbitrary, and the second moment lives in
        # their basis: the factors (a bias of 16 entries gains one rank per step) get twenty steps to
        # become full rank before the first refresh.
        "eigenvalue_corrected": dict(
            grafting_config=ob.AdamPreconditionerConfig(), preconditioner_config=ob.EigenvalueCorrectedShampooPreconditionerConfig(),
            precondition_frequency=20, start_preconditioning_step=20, steps=24,
        ),
        "eigenvalue_corrected_qr": dict(
            preconditioner_config=ob.EigenvalueCorrectedShampooPreconditionerConfig(
                amortized_computation_config=ob.QREigendecompositionConfig(max_iterations=3)
            ),
            precondition_frequency=20, start_preconditioning_step=20, steps=26,
        ),
        "eigenvalue_corrected_exponent_per_order": dict(
            grafting_config=ob.AdamPreconditionerConfig(),
            preconditioner_config=ob.EigenvalueCorrectedShampooPreconditionerConfig(inverse_exponent_override={1: 1.0, 2: 0.25}),
            precondition_frequency=20, start_preconditioning_step=20, steps=24,
        ),
        "rows_only": dict(
            grafting_config=ob.AdamPreconditionerConfig(),
            preconditioner_config=ob.RootInvShampooPreconditionerConfig(inverse_exponent_override={2: {0: 0.25, 1: 0.0}}),
        ),
        "columns_only": dict(
            grafting_config=ob.AdamPreconditionerConfig(),
            preconditioner_config=ob.RootInvShampooPreconditionerConfig(inverse_exponent_override={2: {0: 0.0, 1: 0.5}}),
        ),
        "nothing_preconditioned": dict(
            grafting_config=ob.AdamPreconditionerConfig(),
            preconditioner_config=ob.RootInvShampooPreconditionerConfig(inverse_exponent_override={1: 0.0, 2: 0.0}),
        ),
        "kl_rows_only": dict(
            grafting_config=ob.AdamPreconditionerConfig(),
            preconditioner_config=ob.RootInvKLShampooPreconditionerConfig(inverse_exponent_override={2: {0: 0.5, 1: 0.0}}),
        ),
        "kl_columns_only_vectors_off": dict(
            preconditioner_config=ob.EigendecomposedKLShampooPreconditionerConfig(inverse_exponent_override={1: 0.0, 2: {0: 0.0, 1: 0.5}}),
        ),
        "coupled_newton": dict(
            grafting_config=ob.AdamPreconditionerConfig(), epsilon=1e-4,
            preconditioner_config=ob.RootInvShampooPreconditionerConfig(amortized_computation_config=ob.CoupledNewtonConfig(tolerance=1e-6)),
        ),
    }


@pytest.mark.parametrize("name", list(_configs()))
def test_engine_on_the_stand_in_matches_the_torch_step(cpu_engine, name):
    kw = dict(_configs()[name])
    steps = kw.pop("steps", 8)
    visits = (4, 6) if name == "primal_averaging" else ()
    want, _ = _train("torch", steps=steps, visit_eval_at=visits, **kw)
    got, opt = _train("native", steps=steps, visit_eval_at=visits, **kw)
    for rec in opt._per_group_state_lists:
        assert rec["native_engine"] is not None
        rec["native_engine"].check_status()
    assert cpu_engine.gemm_launches > 0 or name == "nothing_preconditioned"
    for a_list, b_list in zip(want, got, strict=True):
        for a, b in zip(a_list, b_list):
            loose = name.startswith("eigenvalue_corrected")  # eigenvectors react to the last bits of the factors
            assert torch.allclose(a, b, rtol=1e-4, atol=2e-4 if loose else 2e-6), (name, (a - b).abs().max().item())


def test_engine_with_a_gradient_that_goes_missing(cpu_engine):
    kw = dict(grafting_config=ob.AdamPreconditionerConfig(), weight_decay=1e-2)
    want, _ = _train("torch", drop_grad_at=(2, 5), **kw)
    got, _ = _train("native", drop_grad_at=(2, 5), **kw)
    for a, b in zip(want[-1], got[-1]):
        assert torch.allclose(a, b, rtol=1e-4, atol=2e-6), (a - b).abs().max().item()


# ----------------------------------------------------------------------------------------------
# The same under the DDP distributor, ranks as gloo processes
# ----------------------------------------------------------------------------------------------
_scenario_runs: dict = {}


def _every_mode(rank, world, worker, args, modes):
    """Inside one rank: the scenario under each mode in turn (the torch step first; the stand-ins a
    native mode installs leave the torch step alone)."""
    return {mode: worker(rank, world, *args, mode) for mode in modes}


def _scenario(worker, world, args, modes):
    """Per-rank results of ``worker(rank, world, *args, mode)`` for every mode, from one set of spawned
    ranks per scenario however many tests look at it: starting the ranks costs more than the steps."""
    from dist_utils_for_tests import run_distributed

    key = (worker.__name__, world, args)
    if key not in _scenario_runs:
        per_rank = run_distributed(_every_mode, world, worker, args, modes)
        _scenario_runs[key] = {mode: [rank_result[mode] for rank_result in per_rank] for mode in modes}
    assert set(modes) <= set(_scenario_runs[key]), "a scenario is always asked for with the same modes"
    return _scenario_runs[key]


def _ddp_worker(rank, world, case, backend):
    import optimizers_b200 as lib

    if backend == "native":
        install_cpu_engine(setattr)
    torch.manual_seed(0)
    if case == "one_block":
        # a single block: every rank but its owner is idle, and still gathers and applies
        model = torch.nn.Sequential(torch.nn.Linear(12, 8, bias=False))
    else:
        model = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.Tanh(), torch.nn.Linear(20, 8), torch.nn.Linear(8, 8))
    comm = torch.bfloat16 if case == "bf16" else torch.float32
    opt = lib.DistributedShampoo(
        model.parameters(), lr=1e-2, betas=(0.9, 0.999), epsilon=1e-4, max_preconditioner_dim=16, precondition_frequency=3,
        start_preconditioning_step=3, weight_decay=1e-2, grafting_config=lib.AdamPreconditionerConfig(),
        distributed_config=lib.DDPDistributedConfig(
            communication_dtype=comm, num_trainers_per_group=world, communicate_params=case == "communicate_params"
        ),
        native_runtime_config=lib.NativeRuntimeConfig(backend=backend),
    )
    if backend == "native":
        assert all(rec["native_engine"] is not None for rec in opt._per_group_state_lists)
    g = torch.Generator().manual_seed(5)
    for step in range(7):
        x = torch.randn(16, 12, generator=g)
        opt.zero_grad(set_to_none=True)
        if case == "dead_layer":
            out = model[2](model[1](model[0](x)))  # the last layer never gets a gradient
        else:
            out = model(x)
        out.square().mean().backward()
        if case == "missing_grads" and step % 2 == 1:
            list(model.parameters())[0].grad = None
        opt.step()
    return [p.detach().clone() for p in model.parameters()]


@pytest.mark.parametrize(
    "case,world", [("plain", 2), ("plain", 3), ("bf16", 2), ("communicate_params", 2), ("one_block", 3), ("dead_layer", 2), ("missing_grads", 2)]
)
def test_engine_under_ddp_matches_the_torch_step_on_every_rank(case, world):
    """Block ownership, the send slots, the all-gather and the gathered apply of the engine under the
    DDP distributor, with the communication dtypes of the benchmarks, idle ranks, a layer without
    gradients and gradients that vanish on some steps: the same parameters as the torch step, on
    every rank."""
    from dist_utils_for_tests import run_distributed

    runs = _scenario(_ddp_worker, world, (case,), ("torch", "native"))
    want, got = runs["torch"], runs["native"]
    for ref_rank, twin_rank in zip(want, got, strict=True):
        for a, b in zip(ref_rank, twin_rank, strict=True):
            assert torch.allclose(a, b, rtol=1e-4, atol=2e-6), (case, (a - b).abs().max().item())
    for other in got[1:]:
        for a, b in zip(got[0], other):
            assert torch.equal(a, b), "ranks diverged"


# ----------------------------------------------------------------------------------------------
# ... and under the sharded distributors
# ----------------------------------------------------------------------------------------------
_P2P_SHARDED = [("hsdp", 4), ("hsdp", 8), ("hybrid_shard", 4), ("fully_shard:ROUND_ROBIN", 2), ("hybrid_shard:ROUND_ROBIN", 4)]


def _sharded_modes(strategy, world):
    """The torch step, the engine over the collectives and, where the strategy has one, the engine
    over peer memory (the eight-rank layout is run for that form only)."""
    if (strategy, world) == ("hsdp", 8):
        return ("torch", "native_p2p")
    return ("torch", "native", "native_p2p") if (strategy, world) in _P2P_SHARDED else ("torch", "native")


def _sharded_worker(rank, world, strategy, backend):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, ShardingStrategy, fully_shard
    from torch.distributed.tensor import DTensor

    import optimizers_b200 as lib

    if backend != "torch":
        install_cpu_engine(setattr)
    if backend == "native_p2p":
        import torch.distributed._symmetric_memory as symm_mem

        import fake_peers
        from optimizers_b200.ops import build

        import optimizers_b200.parallel.a2a as a2a

        ext = fake_peers.FakePeerExt()
        build.load = lambda: ext
        symm_mem.empty = fake_peers.symm_empty
        symm_mem.rendezvous = fake_peers.symm_rendezvous
        torch.cuda.synchronize = lambda device=None: None
        a2a._PEER_DEVICE_TYPES = ("cuda", "cpu")
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.Tanh(), torch.nn.Linear(20, 8), torch.nn.Tanh(), torch.nn.Linear(8, 4))
    cpu = torch.device("cpu")
    kind, _, assignment = strategy.partition(":")
    extra = {} if not assignment else dict(param_assignment_strategy=lib.FSDPParamAssignmentStrategy[assignment])
    if kind == "fsdp":
        model = FSDP(model, use_orig_params=True, device_id=cpu)
        cfg = lib.FSDPDistributedConfig(param_to_metadata=lib.compile_fsdp_parameter_metadata(model))
    elif kind == "hsdp":
        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
        model = FSDP(model, device_mesh=mesh, sharding_strategy=ShardingStrategy.HYBRID_SHARD, use_orig_params=True, device_id=cpu)
        cfg = lib.HSDPDistributedConfig(param_to_metadata=lib.compile_fsdp_parameter_metadata(model), device_mesh=mesh)
    elif kind == "fully_shard":
        fully_shard(model, mesh=init_device_mesh("cpu", (world,)))
        cfg = lib.FullyShardDistributedConfig(**extra)
    else:
        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("replicate", "shard"))
        fully_shard(model, mesh=mesh)
        cfg = lib.HybridShardDistributedConfig(device_mesh=mesh, **extra)
    opt = lib.DistributedShampoo(
        model.parameters(), lr=1e-2, betas=(0.9, 0.999), epsilon=1e-4, max_preconditioner_dim=8, precondition_frequency=3,
        start_preconditioning_step=3, weight_decay=1e-2, grafting_config=lib.AdamPreconditionerConfig(), distributed_config=cfg,
        native_runtime_config=lib.NativeRuntimeConfig(
            backend="torch" if backend == "torch" else "native", comm_path="p2p" if backend == "native_p2p" else "nccl"
        ),
    )
    engines = [rec.get("native_engine") for rec in opt._per_group_state_lists]
    g = torch.Generator().manual_seed(5)
    for _ in range(7):
        x, y = torch.randn(16, 12, generator=g), torch.randint(0, 4, (16,), generator=g)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    if backend == "native_p2p":
        for rec, engine in zip(opt._per_group_state_lists, engines):
            d = rec["distributor"]
            if getattr(d, "_gather_grads_ctx", None) is not None:  # lossless: the all-to-all contexts own the arenas
                for ctx in (d._gather_grads_ctx, d._redistribute_ctx):
                    if ctx._group_size > 1:
                        assert ctx._p2p and ctx._arena.overrun_regions() == []
                    ctx.check_status()
            else:
                assert engine._p2p and engine._arena.overrun_regions() == []
            engine.check_status()
    local = [(p.to_local() if isinstance(p, DTensor) else p).detach().clone() for p in model.parameters()]
    return local, [e is not None for e in engines]


@pytest.mark.parametrize(
    "strategy,world",
    [("fsdp", 2), ("hsdp", 4), ("fully_shard", 2), ("fully_shard:ROUND_ROBIN", 2), ("fully_shard:REPLICATE", 2),
     ("hybrid_shard", 4), ("hybrid_shard:ROUND_ROBIN", 4)],
)
def test_engine_under_the_sharded_distributors_matches_the_torch_step(strategy, world):
    """Flat shards with recovered blocks (FSDP1 / HSDP1), dim-0 shards, the lossless variants' full
    copies with their all-to-all write-back, and the replicate-group all-gather of the hybrid forms."""
    from dist_utils_for_tests import run_distributed

    runs = _scenario(_sharded_worker, world, (strategy,), _sharded_modes(strategy, world))
    want, got = runs["torch"], runs["native"]
    for (ref_rank, _), (twin_rank, engines) in zip(want, got, strict=True):
        assert all(engines), "the engine was not built on every rank"
        for a, b in zip(ref_rank, twin_rank, strict=True):
            assert a.shape == b.shape and torch.allclose(a, b, rtol=1e-4, atol=2e-6), (strategy, (a - b).abs().max().item())


# ----------------------------------------------------------------------------------------------
# Convolution weights (order-3 blocks), checkpoints, mode switches across ranks
# ----------------------------------------------------------------------------------------------
def _conv_train(backend, steps=7, **kw):
    torch.manual_seed(0)
    model = torch.nn.Sequential(
        torch.nn.Conv2d(4, 16, 3, padding=1, bias=False), torch.nn.ReLU(), torch.nn.Conv2d(16, 8, 3, padding=1),
        torch.nn.AdaptiveAvgPool2d(1), torch.nn.Flatten(), torch.nn.Linear(8, 3),
    )
    args = dict(lr=1e-2, betas=(0.9, 0.999), epsilon=1e-4, max_preconditioner_dim=16, precondition_frequency=3,
                start_preconditioning_step=3, grafting_config=ob.AdamPreconditionerConfig(), weight_decay=1e-2)
    args.update(kw)
    opt = ob.DistributedShampoo(model.parameters(), native_runtime_config=ob.NativeRuntimeConfig(backend=backend), **args)
    g = torch.Generator().manual_seed(2)
    for _ in range(steps):
        x, y = torch.randn(8, 4, 6, 6, generator=g), torch.randint(0, 3, (8,), generator=g)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    return [p.detach().clone() for p in model.parameters()], opt


def test_engine_on_convolution_weights_with_eigenvalue_correction(cpu_engine):
    """Order-3 blocks under eigenvalue-corrected Shampoo: the raw and the filtered gradient are
    projected through the three eigenbases side by side, the second moment is taken in the
    eigenbasis, and the scaled direction goes back through the three bases.  The first refresh
    waits until the factors have full rank (see the 2-D case above)."""
    kw = dict(preconditioner_config=ob.EigenvalueCorrectedShampooPreconditionerConfig(), precondition_frequency=20,
              start_preconditioning_step=20)
    want, _ = _conv_train("torch", steps=24, **kw)
    got, opt = _conv_train("native", steps=24, **kw)
    engine = opt._per_group_state_lists[0]["native_engine"]
    assert engine is not None and any(b.dims3 is not None for b in engine._blocks)
    for a, b in zip(want, got):
        assert torch.allclose(a, b, rtol=1e-4, atol=2e-5), (a - b).abs().max().item()


@pytest.mark.parametrize("eigdec", [False, True])
def test_engine_on_convolution_weights_matches_the_torch_step(cpu_engine, eigdec):
    """(16, 4, 3, 3) and (8, 16, 3, 3) weights become order-3 tensors (out, in, kh * kw) with out and in
    multiples of 4: the three mode unfoldings, the auxiliary descriptor of the second view and
    the three chained products."""
    kw = dict(preconditioner_config=ob.EigendecomposedShampooPreconditionerConfig()) if eigdec else {}
    want, _ = _conv_train("torch", **kw)
    got, opt = _conv_train("native", **kw)
    engine = opt._per_group_state_lists[0]["native_engine"]
    assert engine is not None and any(b.dims3 is not None for b in engine._blocks)
    for a, b in zip(want, got):
        assert torch.allclose(a, b, rtol=1e-4, atol=2e-6), (a - b).abs().max().item()


def test_engine_resumes_from_a_checkpoint(cpu_engine):
    """A fresh optimizer that loads the state of a running one continues exactly like it: the operand
    mirrors of the inverse roots are rebuilt from the loaded state."""
    import copy

    kw = dict(grafting_config=ob.AdamPreconditionerConfig(), weight_decay=1e-2)

    def build(model):
        return ob.DistributedShampoo(
            model.parameters(), lr=1e-2, betas=(0.9, 0.999), epsilon=1e-4, max_preconditioner_dim=16, precondition_frequency=3,
            start_preconditioning_step=3, native_runtime_config=ob.NativeRuntimeConfig(backend="native"), **kw
        )

    def steps(model, opt, generator, count):
        for _ in range(count):
            x, y = torch.randn(32, 20, generator=generator), torch.randint(0, 4, (32,), generator=generator)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()

    model = _model()
    opt = build(model)
    g = torch.Generator().manual_seed(1)
    steps(model, opt, g, 5)
    saved_model, saved_opt, saved_rng = copy.deepcopy(model.state_dict()), copy.deepcopy(opt.state_dict()), g.get_state()
    steps(model, opt, g, 4)

    resumed = _model()
    resumed.load_state_dict(saved_model)
    resumed_opt = build(resumed)
    resumed_opt.load_state_dict(saved_opt)
    g2 = torch.Generator()
    g2.set_state(saved_rng)
    steps(resumed, resumed_opt, g2, 4)
    for a, b in zip(model.parameters(), resumed.parameters()):
        assert torch.equal(a, b), (a - b).abs().max().item()


def _gpa_ddp_worker(rank, world, backend):
    import optimizers_b200 as lib

    if backend == "native":
        install_cpu_engine(setattr)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.Tanh(), torch.nn.Linear(20, 8))
    opt = lib.DistributedShampoo(
        model.parameters(), lr=1e-2, betas=(0.9, 0.999), epsilon=1e-4, max_preconditioner_dim=16, precondition_frequency=3,
        start_preconditioning_step=3, weight_decay=1e-2, grafting_config=lib.AdamPreconditionerConfig(),
        iterate_averaging_config=lib.GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.9, train_interp_coeff=0.7),
        distributed_config=lib.DDPDistributedConfig(communication_dtype=torch.float32, num_trainers_per_group=world),
        native_runtime_config=lib.NativeRuntimeConfig(backend=backend),
    )
    opt.train()
    g = torch.Generator().manual_seed(5)
    seen = []
    for step in range(7):
        if step in (4, 6):
            opt.eval()
            seen.append([p.detach().clone() for p in model.parameters()])
            opt.train()
        x = torch.randn(16, 12, generator=g)
        opt.zero_grad()
        model(x).square().mean().backward()
        opt.step()
    opt.eval()
    seen.append([p.detach().clone() for p in model.parameters()])
    return seen


def test_engine_mode_switches_under_ddp_match_the_torch_step():
    """train() / eval() of primal averaging with block ownership spread over ranks: every rank
    switches every parameter (the owners' deltas travel through the all-gather buffer)."""
    from dist_utils_for_tests import run_distributed

    runs = _scenario(_gpa_ddp_worker, 2, (), ("torch", "native"))
    want, got = runs["torch"], runs["native"]
    for ref_rank, twin_rank in zip(want, got, strict=True):
        for a_list, b_list in zip(ref_rank, twin_rank, strict=True):
            for a, b in zip(a_list, b_list):
                assert torch.allclose(a, b, rtol=1e-4, atol=2e-6), (a - b).abs().max().item()


@pytest.mark.parametrize("scenario", ["corrected_weight_decay_momentum", "schedule_free", "two_groups"])
def test_engine_with_a_learning_rate_schedule_and_parameter_groups(cpu_engine, scenario):
    """The learning rate is a device scalar refreshed every step: the corrected weight decay, the
    Schedule-Free weights and the epilogue's ``-lr`` must follow a schedule; two groups get two engines."""

    def run(backend):
        model = _model()
        params = list(model.parameters())
        kw = dict(lr=2e-2, betas=(0.9, 0.999), epsilon=1e-4, max_preconditioner_dim=16, precondition_frequency=3,
                  start_preconditioning_step=3, grafting_config=ob.AdamPreconditionerConfig())
        groups = params
        if scenario == "corrected_weight_decay_momentum":
            kw.update(weight_decay=0.05, weight_decay_type=ob.WeightDecayType.CORRECTED,
                      iterate_averaging_config=ob.ClassicMomentumConfig(momentum=0.8, dampening=0.0, use_nesterov=True))
        elif scenario == "schedule_free":
            kw.update(iterate_averaging_config=ob.ScheduleFreeConfig(train_interp_coeff=0.9), weight_decay=0.01)
        else:
            groups = [dict(params=params[:2], lr=1e-2), dict(params=params[2:], weight_decay=0.02, max_preconditioner_dim=8)]
        opt = ob.DistributedShampoo(groups, native_runtime_config=ob.NativeRuntimeConfig(backend=backend), **kw)
        opt.train()
        g = torch.Generator().manual_seed(1)
        for step in range(9):
            for group in opt.param_groups:
                group["lr"] = group["lr"] * (1.3 if step < 3 else 0.8)
            x, y = torch.randn(32, 20, generator=g), torch.randint(0, 4, (32,), generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
        opt.eval()
        return [p.detach().clone() for p in model.parameters()], opt

    want, _ = run("torch")
    got, opt = run("native")
    assert all(rec["native_engine"] is not None for rec in opt._per_group_state_lists)
    for a, b in zip(want, got):
        assert torch.allclose(a, b, rtol=1e-4, atol=2e-6), (scenario, (a - b).abs().max().item())


# ----------------------------------------------------------------------------------------------
# The peer-memory paths, with shared memory standing in for NVLink peers
# ----------------------------------------------------------------------------------------------
def _p2p_worker(rank, world, case, mode):
    import torch.distributed._symmetric_memory as symm_mem

    import fake_peers
    import optimizers_b200 as lib
    import optimizers_b200.native_engine as engine_module
    from optimizers_b200.ops import build

    if mode != "torch":
        install_cpu_engine(setattr)
        ext = fake_peers.FakePeerExt()
        build.load = lambda: ext
        symm_mem.empty = fake_peers.symm_empty
        symm_mem.rendezvous = fake_peers.symm_rendezvous
        torch.cuda.synchronize = lambda device=None: None
    torch.manual_seed(0)
    if case == "one_block":
        model = torch.nn.Sequential(torch.nn.Linear(12, 8, bias=False))
    else:
        model = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.Tanh(), torch.nn.Linear(20, 8), torch.nn.Linear(8, 8))
    pull = mode == "p2p_pull"
    train_model = model if pull else torch.nn.parallel.DistributedDataParallel(model)
    opt = lib.DistributedShampoo(
        model.parameters(), lr=1e-2, betas=(0.9, 0.999), epsilon=1e-4, max_preconditioner_dim=16, precondition_frequency=3,
        start_preconditioning_step=3, weight_decay=1e-2, grafting_config=lib.AdamPreconditionerConfig(),
        distributed_config=lib.DDPDistributedConfig(
            communication_dtype=torch.bfloat16 if case == "bf16" else torch.float32, num_trainers_per_group=world
        ),
        native_runtime_config=lib.NativeRuntimeConfig(
            backend="torch" if mode == "torch" else "native", comm_path="nccl" if mode == "torch" else "p2p",
            fuse_gradient_reduction=pull, fuse_direction_push=mode == "p2p_gemm",
        ),
    )
    if mode != "torch":
        engine = opt._per_group_state_lists[0]["native_engine"]
        assert engine is not None and engine._p2p and engine._pull == pull
    g = torch.Generator().manual_seed(5)
    for _ in range(7):
        x = torch.randn(16, 12, generator=g)
        shard = slice(rank * 16 // world, (rank + 1) * 16 // world)
        opt.zero_grad(set_to_none=not pull)
        loss = train_model(x[shard]).square().mean()
        loss.backward()
        opt.step()
    if mode != "torch":
        assert engine._arena.overrun_regions() == []
        engine.check_status()
        # 7 steps, preconditioning from step 3: five steps gather from the epilogue of the last product
        assert engine.gemm_push_steps == (5 if (mode == "p2p_gemm" and engine._blocks) else 0)  # a rank without blocks pushes nothing
    return [p.detach().clone() for p in model.parameters()]


@pytest.mark.parametrize("mode", ["p2p_push", "p2p_pull", "p2p_gemm"])
@pytest.mark.parametrize("case,world", [("plain", 2), ("plain", 3), ("bf16", 2), ("one_block", 3)])
def test_engine_peer_memory_paths_match_the_torch_step(case, world, mode):
    """The all-gather by peer stores from the epilogue and the gradient reduction by peer loads in the
    prologue (which replaces torch's DDP wrapper), with the engine's own barriers between them, over
    memory shared between the ranks: the same parameters as the torch step under torch DDP, on every
    rank, and the arena's guard regions intact."""
    from dist_utils_for_tests import run_distributed

    runs = _scenario(_p2p_worker, world, (case,), ("torch", "p2p_push", "p2p_pull", "p2p_gemm"))
    want, got = runs["torch"], runs[mode]
    # The GEMM-epilogue form rounds the unscaled direction to the communication dtype and scales on
    # the receiving side; the other forms round the finished update: in bf16 they differ by its rounding.
    atol = 5e-4 if (case == "bf16" and mode == "p2p_gemm") else 2e-6
    for ref_rank, twin_rank in zip(want, got, strict=True):
        for a, b in zip(ref_rank, twin_rank, strict=True):
            assert torch.allclose(a, b, rtol=1e-4, atol=atol), (case, mode, (a - b).abs().max().item())
    for other in got[1:]:
        for a, b in zip(got[0], other):
            assert torch.equal(a, b), "ranks diverged"



def test_engine_peer_memory_paths_on_eight_ranks():
    """The DDP arm of the flagship benchmark on eight GPUs: bf16 directions, gradients reduced by peer
    loads in the prologue, directions gathered by peer stores, eight ranks sharing nine blocks (one rank
    owns two)."""
    from dist_utils_for_tests import run_distributed

    runs = _scenario(_p2p_worker, 8, ("bf16",), ("torch", "p2p_pull"))
    want, got = runs["torch"], runs["p2p_pull"]
    for ref_rank, twin_rank in zip(want, got, strict=True):
        for a, b in zip(ref_rank, twin_rank, strict=True):
            assert torch.allclose(a, b, rtol=1e-4, atol=2e-6), (a - b).abs().max().item()
    for other in got[1:]:
        for a, b in zip(got[0], other):
            assert torch.equal(a, b), "ranks diverged"


@pytest.mark.parametrize(
    "strategy,world",
    _P2P_SHARDED,  # ("hsdp", 8) is the layout of the flagship benchmark on eight GPUs: replicate 2 x shard 4
)
def test_engine_peer_memory_paths_under_the_sharded_distributors(strategy, world):
    """``comm_path="p2p"`` beyond plain DDP: the replicate groups of HSDP / hybrid shard gather the
    directions by peer stores within their sub-group (the flag barrier spans that sub-group only), and
    the lossless ROUND_ROBIN exchange moves gradients and parameters by grouped peer copies."""
    from dist_utils_for_tests import run_distributed

    runs = _scenario(_sharded_worker, world, (strategy,), _sharded_modes(strategy, world))
    want, got = runs["torch"], runs["native_p2p"]
    for (ref_rank, _), (twin_rank, engines) in zip(want, got, strict=True):
        assert all(engines)
        for a, b in zip(ref_rank, twin_rank, strict=True):
            assert a.shape == b.shape and torch.allclose(a, b, rtol=1e-4, atol=2e-6), (strategy, (a - b).abs().max().item())


def _departing_rank_worker(rank, world):
    import time

    import torch.distributed._symmetric_memory as symm_mem

    import fake_peers
    import optimizers_b200 as lib
    from optimizers_b200.ops import build

    install_cpu_engine(setattr)
    ext = fake_peers.FakePeerExt()
    ext.barrier_timeout = 1.0
    build.load = lambda: ext
    symm_mem.empty = fake_peers.symm_empty
    symm_mem.rendezvous = fake_peers.symm_rendezvous
    torch.cuda.synchronize = lambda device=None: None
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.Tanh(), torch.nn.Linear(20, 8))
    opt = lib.DistributedShampoo(
        model.parameters(), lr=1e-2, epsilon=1e-4, max_preconditioner_dim=16, precondition_frequency=3, start_preconditioning_step=3,
        grafting_config=lib.AdamPreconditionerConfig(),
        distributed_config=lib.DDPDistributedConfig(communication_dtype=torch.float32, num_trainers_per_group=world),
        native_runtime_config=lib.NativeRuntimeConfig(backend="native", comm_path="p2p", fuse_gradient_reduction=True),
    )
    engine = opt._per_group_state_lists[0]["native_engine"]
    g = torch.Generator().manual_seed(5)

    def step():
        opt.zero_grad(set_to_none=False)
        model(torch.randn(8, 12, generator=g)).square().mean().backward()
        opt.step()

    step()
    step()
    if rank == 1:
        time.sleep(3.0)  # leaves between steps; stays alive until the other rank has given up waiting
        return "left"
    before = [p.detach().clone() for p in model.parameters()]
    start = time.monotonic()
    try:
        step()  # the entry barrier runs out: the status word gets the peer-timeout bit
        waited = time.monotonic() - start
        engine.check_status()  # (a refresh step checks the word itself and raises from inside the step)
    except RuntimeError as error:
        waited = time.monotonic() - start
        unchanged = all(torch.equal(a, b) for a, b in zip(before, model.parameters()))
        return ("raised", str(error), waited, unchanged)
    return ("silent", "", waited, False)


def test_a_rank_that_leaves_is_reported_by_the_bounded_peer_wait():
    """Failure made on the host: one rank stops stepping.  The other's flag wait runs out after its
    limit, the status word carries the peer-timeout bit, ``check_status`` raises, and the parameters
    were left as they were (the gathered apply skips its update when that bit is set)."""
    from dist_utils_for_tests import run_distributed

    results = run_distributed(_departing_rank_worker, 2)
    assert results[1] == "left"
    outcome, message, waited, unchanged = results[0]
    assert outcome == "raised", results[0]
    assert "peer" in message.lower()
    assert 0.9 < waited < 10.0
    assert unchanged


@pytest.mark.parametrize("gemm_mode", ["tf32x3", "tf32"])
def test_memory_report_counts_every_array_once(cpu_engine, gemm_mode):
    """The engine's own account of its device memory: checked by hand for one 20 x 36 weight cut
    into 16-wide blocks.  With split (hi, lo) operands a block m x n holds G, G^T and the filtered
    gradient twice each (the direction and the chain intermediate live in G and G^T) and its two
    inverse roots twice; a single-pass tf32 configuration holds half of that."""
    torch.manual_seed(0)
    layer = torch.nn.Linear(36, 20, bias=False)
    opt = ob.DistributedShampoo(
        layer.parameters(), lr=1e-2, epsilon=1e-4, max_preconditioner_dim=16, precondition_frequency=3,
        native_runtime_config=ob.NativeRuntimeConfig(backend="native", gemm_mode=gemm_mode),
    )
    (report,) = opt.native_memory_report()
    copies = 2 if gemm_mode == "tf32x3" else 1
    pad = lambda n: (n + 3) // 4 * 4  # noqa: E731
    operands = mirrors = state = 0
    for m in (16, 4):
        for n in (16, 16, 4):
            operands += copies * 4 * (2 * m * pad(n) + n * pad(m))
            mirrors += copies * 4 * (m * pad(m) + n * pad(n))
            # packed factors and inverse roots, filtered gradient (no grafting, no momentum)
            state += 4 * (2 * (m * (m + 1) // 2 + n * (n + 1) // 2) + m * n)
    assert report["operands"] == operands
    assert report["mirrors"] == mirrors
    assert report["state"] == state
    assert report["exchange"] == 0 and report["total"] == operands + mirrors + state
    torch_only = ob.DistributedShampoo(layer.parameters(), native_runtime_config=ob.NativeRuntimeConfig(backend="torch"))
    assert torch_only.native_memory_report() == [None]


def test_engine_keeps_the_filtered_gradient_apart_from_the_direction(cpu_engine):
    """Without bias correction the reference's applied filtered gradient is the state tensor itself,
    and with SGD grafting before preconditioning starts the search direction is that tensor too: its
    in-place scaling by -lr ends up in the state (the torch step reproduces this, bit for bit).  The
    engine's prologue writes the moving average and the direction to different arrays."""
    stored = {}
    for backend in ("torch", "native"):
        p = torch.nn.Parameter(torch.zeros(3, 3))
        opt = ob.DistributedShampoo(
            [p], lr=0.1, betas=(0.9, 1.0), epsilon=1e-3, use_bias_correction=False, grafting_config=ob.SGDPreconditionerConfig(),
            precondition_frequency=2, start_preconditioning_step=4, max_preconditioner_dim=16,
            native_runtime_config=ob.NativeRuntimeConfig(backend=backend),
        )
        p.grad = torch.ones(3, 3)
        opt.step()
        stored[backend] = opt.state_dict()["state"][0]["block_0"]["filtered_grad"].flatten()[0].item()
        assert p.flatten()[0].item() == pytest.approx(-0.01)  # the same update either way
    assert stored["torch"] == pytest.approx(-0.01)  # the reference's write-through
    assert stored["native"] == pytest.approx(0.1)  # the moving average of a gradient of 1 from 0


def test_engine_on_random_option_sets_matches_the_torch_step(cpu_engine):
    """Thirty random option sets of the families whose result does not hinge on the choice of
    eigenvectors inside a null space (root-inverse by eigendecomposition and by coupled Newton,
    eigendecomposed, both KL forms), with random grafting, betas, weight decay, averaging, block
    size, schedule, exponent overrides and GEMM mode: the engine ends where the torch step ends.
    Option sets in which the reference lets the search direction write through to the
    filtered-gradient state get bias correction switched on (the engine deliberately does not
    reproduce that; see test_engine_keeps_the_filtered_gradient_apart_from_the_direction)."""
    import logging
    import math
    import random

    import test_random_option_sets_parity as option_sets

    def train(backend, seed):
        rng = random.Random(seed)
        while True:
            family, kw = option_sets._options(ob, rng)
            if family in ("root_inv", "root_inv_newton", "eigendecomposed", "kl_root_inv", "kl_eigendecomposed"):
                break
        kw["epsilon"] = max(kw["epsilon"], 1e-3)
        if kw["max_preconditioner_dim"] == math.inf:
            kw["max_preconditioner_dim"] = 32
        identity_blocks = getattr(kw["preconditioner_config"], "inverse_exponent_override", {}).get(1) == 0.0
        if type(kw.get("grafting_config")).__name__ in ("SGDPreconditionerConfig", "NoneType") or identity_blocks:
            kw["use_bias_correction"] = True
        runtime = ob.NativeRuntimeConfig(backend=backend, gemm_mode=rng.choice(["tf32x3", "tf32"]))
        torch.manual_seed(seed)
        if rng.random() < 0.3:
            model = torch.nn.Sequential(torch.nn.Conv2d(2, 4, 3), torch.nn.Flatten(), torch.nn.Linear(4 * 4 * 4, 3))
            shape = (32, 2, 6, 6)
        else:
            model = torch.nn.Sequential(torch.nn.Linear(9, 12), torch.nn.Tanh(), torch.nn.Linear(12, 3, bias=False))
            shape = (32, 9)
        try:
            opt = ob.DistributedShampoo(model.parameters(), native_runtime_config=runtime, **kw)
        except RuntimeError:
            return None  # not covered natively (backend="native" says so instead of falling back)
        g = torch.Generator().manual_seed(seed + 1)
        opt.train()
        for step in range(7):
            x, y = torch.randn(*shape, generator=g), torch.randint(0, 3, (shape[0],), generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
            if step == 4:
                opt.eval()
                opt.train()
        opt.eval()
        return [p.detach().clone() for p in model.parameters()]

    logging.disable(logging.WARNING)
    try:
        compared = 0
        for seed in range(30):
            got = train("native", seed)
            if got is None:
                continue
            want = train("torch", seed)
            compared += 1
            for a, b in zip(want, got, strict=True):
                assert torch.allclose(a, b, rtol=1e-3, atol=1e-3 * float(a.abs().max())), (seed, (a - b).abs().max().item())
        assert compared >= 15
    finally:
        logging.disable(logging.NOTSET)


def test_native_coverage_names_the_reason_of_a_fallback(monkeypatch):
    """``backend="auto"`` falls back silently; ``native_coverage()`` says per parameter group whether
    the engine runs it and, if not, why (the text ``backend="native"`` would raise with)."""
    import optimizers_b200.native_engine as engine_module
    from optimizers_b200.ops import build

    layer = torch.nn.Linear(6, 4)
    assert ob.DistributedShampoo(layer.parameters()).native_coverage() == ["torch: the parameters are not on a CUDA device"]
    forced = ob.DistributedShampoo(layer.parameters(), native_runtime_config=ob.NativeRuntimeConfig(backend="torch"))
    assert forced.native_coverage() == ['torch: backend="torch" was requested']

    # the engine's own decision, on CPU parameters through the stand-in of the extension
    install_cpu_engine(monkeypatch.setattr)
    monkeypatch.setattr(engine_module, "maybe_build_native_engine", engine_module.build_native_engine)
    assert build.available()
    covered = ob.DistributedShampoo(layer.parameters(), max_preconditioner_dim=8)
    assert covered.native_coverage() == ["native"]
    groups = [
        {"params": [layer.weight]},
        {"params": [layer.bias], "preconditioner_config": ob.DefaultSignDescentPreconditionerConfig},
    ]
    mixed = ob.DistributedShampoo(groups, max_preconditioner_dim=8)
    first, second = mixed.native_coverage()
    assert first == "native"
    assert second == "torch: preconditioner config SignDescentPreconditionerConfig has no native step yet"
    assert mixed.native_memory_report()[1] is None
