"""Optimizer-level behaviour: equivalences with torch.optim, agreement with the reference on
every preconditioner family, state-dict layout, train/eval modes, validation."""

import copy
import math

import pytest
import torch

import optimizers_b200 as ob
from ref_oracle import reference, reference_available


def _model(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(10, 12), torch.nn.ReLU(), torch.nn.Linear(12, 6, bias=False), torch.nn.ReLU(), torch.nn.Linear(6, 3))


def _batches(n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(16, 10, generator=g), torch.randint(0, 3, (16,), generator=g)) for _ in range(n)]


def _run(make_opt, steps=6, model=None, skip_grad_of=None):
    model = model or _model()
    opt = make_opt(model.parameters())
    if hasattr(opt, "train"):
        opt.train()
    losses = []
    for x, y in _batches(steps):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        if skip_grad_of is not None:
            list(model.parameters())[skip_grad_of].grad = None
        opt.step()
        losses.append(loss.item())
    return model, opt, losses


def _assert_same_params(m1, m2, exact=True, **tol):
    for a, b in zip(m1.parameters(), m2.parameters()):
        if exact:
            assert torch.equal(a, b), (a - b).abs().max()
        else:
            torch.testing.assert_close(a, b, **tol)


# --------------------------------------------------------------------------------------------
# Grafting-only Shampoo equals the corresponding torch.optim optimizer
# --------------------------------------------------------------------------------------------
def _shampoo_as(grafting, **kw):
    kw.setdefault("betas", (0.0, 1.0))
    kw.setdefault("use_bias_correction", True)
    return lambda params: ob.DistributedShampoo(
        params, epsilon=1e-10, max_preconditioner_dim=4, precondition_frequency=1,
        start_preconditioning_step=math.inf, grafting_config=grafting, **kw
    )


@pytest.mark.parametrize(
    "torch_opt,ours",
    [
        (lambda p: torch.optim.SGD(p, lr=0.1), _shampoo_as(ob.SGDPreconditionerConfig(), lr=0.1)),
        (lambda p: torch.optim.SGD(p, lr=0.1, weight_decay=0.01),
         _shampoo_as(ob.SGDPreconditionerConfig(), lr=0.1, weight_decay=0.01, weight_decay_type=ob.WeightDecayType.L2)),
        (lambda p: torch.optim.Adagrad(p, lr=0.05, eps=1e-10), _shampoo_as(ob.AdaGradPreconditionerConfig(epsilon=1e-10), lr=0.05)),
        (lambda p: torch.optim.RMSprop(p, lr=0.01, alpha=0.99, eps=1e-8),
         _shampoo_as(ob.RMSpropPreconditionerConfig(beta2=0.99, epsilon=1e-8), lr=0.01, use_bias_correction=False)),
        (lambda p: torch.optim.Adam(p, lr=0.01, betas=(0.9, 0.999), eps=1e-8),
         _shampoo_as(ob.AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8), lr=0.01, betas=(0.9, 0.999))),
        (lambda p: torch.optim.AdamW(p, lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.05),
         _shampoo_as(ob.AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8), lr=0.01, betas=(0.9, 0.999), weight_decay=0.05)),
    ],
    ids=["sgd", "sgd_l2", "adagrad", "rmsprop", "adam", "adamw"],
)
def test_grafting_matches_torch_optim(torch_opt, ours):
    m_ref, _, _ = _run(torch_opt)
    m_our, _, _ = _run(ours)
    _assert_same_params(m_ref, m_our, exact=False, rtol=2e-5, atol=2e-6)


def test_classic_momentum_matches_sgd_momentum():
    for nesterov in (False, True):
        m_ref, _, _ = _run(lambda p: torch.optim.SGD(p, lr=0.1, momentum=0.5, nesterov=nesterov))
        m_our, _, _ = _run(
            _shampoo_as(ob.SGDPreconditionerConfig(), lr=0.1, iterate_averaging_config=ob.ClassicMomentumConfig(momentum=0.5, use_nesterov=nesterov))
        )
        _assert_same_params(m_ref, m_our, exact=False, rtol=1e-5, atol=1e-6)


def test_gpa_reduces_to_plain_steps_and_round_trips_modes():
    cfg = ob.GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.0, train_interp_coeff=1.0)
    m_ref, _, _ = _run(lambda p: torch.optim.SGD(p, lr=0.1))
    m_our, opt, _ = _run(_shampoo_as(ob.SGDPreconditionerConfig(), lr=0.1, iterate_averaging_config=cfg))
    _assert_same_params(m_ref, m_our, exact=False, rtol=1e-5, atol=1e-6)
    # train -> eval -> train returns to the same parameters
    cfg = ob.GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.9, train_interp_coeff=0.7)
    model, opt, _ = _run(_shampoo_as(ob.AdamPreconditionerConfig(), lr=0.01, iterate_averaging_config=cfg))
    before = [p.detach().clone() for p in model.parameters()]
    opt.eval()
    assert any(not torch.equal(a, b) for a, b in zip(before, model.parameters()))
    opt.eval()  # idempotent
    opt.train()
    for a, b in zip(before, model.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    opt.eval()
    with pytest.raises(RuntimeError, match="not in train mode"):
        for p in model.parameters():
            p.grad = torch.ones_like(p)
        opt.step()


def test_gpa_adamw_matches_shampoo_with_adam_preconditioner_and_gpa():
    lr, mu_x, mu_y = 0.01, 0.9, 0.7
    m_gpa, _, _ = _run(lambda p: ob.GPAAdamW(p, lr=lr, eps=1e-8, weight_decay=0.0, train_interp_coeff=mu_y, eval_interp_coeff=mu_x))
    m_shp, _, _ = _run(
        lambda p: ob.DistributedShampoo(
            p, lr=lr, betas=(0.9, 0.999), epsilon=1e-8, max_preconditioner_dim=4, precondition_frequency=1,
            start_preconditioning_step=math.inf, grafting_config=ob.AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8),
            iterate_averaging_config=ob.GeneralizedPrimalAveragingConfig(eval_interp_coeff=mu_x, train_interp_coeff=mu_y),
        )
    )
    _assert_same_params(m_gpa, m_shp, exact=False, rtol=1e-4, atol=1e-5)


# --------------------------------------------------------------------------------------------
# Agreement with the reference implementation (bitwise on CPU)
# --------------------------------------------------------------------------------------------
def _families(lib):
    return {
        "root_inv": dict(preconditioner_config=lib.RootInvShampooPreconditionerConfig()),
        "root_inv_unpacked_newton": dict(
            preconditioner_config=lib.RootInvShampooPreconditionerConfig(
                use_symmetric_packing=False, amortized_computation_config=lib.CoupledNewtonConfig()
            )
        ),
        "root_inv_trace_scaling_override": dict(
            preconditioner_config=lib.RootInvShampooPreconditionerConfig(
                use_trace_scaling=True, inverse_exponent_override={2: {0: 0.5, 1: 0.0}, 1: 0.25}
            )
        ),
        "eigendecomposed": dict(preconditioner_config=lib.EigendecomposedShampooPreconditionerConfig()),
        "eigendecomposed_qr": dict(
            preconditioner_config=lib.EigendecomposedShampooPreconditionerConfig(
                amortized_computation_config=lib.QREigendecompositionConfig(max_iterations=2)
            )
        ),
        "eigenvalue_corrected": dict(preconditioner_config=lib.DefaultEigenvalueCorrectedShampooConfig),
        "soap": dict(preconditioner_config=lib.DefaultSOAPConfig),
        "root_inv_kl": dict(preconditioner_config=lib.RootInvKLShampooPreconditionerConfig()),
        "eigendecomposed_kl": dict(preconditioner_config=lib.EigendecomposedKLShampooPreconditionerConfig()),
        "sign": dict(preconditioner_config=lib.DefaultSignDescentPreconditionerConfig),
        "spectral": dict(
            preconditioner_config=lib.DefaultSpectralDescentPreconditionerConfig,
            max_preconditioner_dim=math.inf,
            distributed_config=lib.SingleDeviceDistributedConfig(target_parameter_dimensionality=2),
        ),
    }


@pytest.mark.skipif(not reference_available(), reason="reference not installed")
@pytest.mark.parametrize("family", list(_families(ob)))
@pytest.mark.parametrize("extras", ["adam_graft_wd", "momentum_beta3", "schedule_free"])
def test_matches_reference_bitwise(family, extras):
    R = reference()

    def build(lib):
        kw = dict(lr=0.02, betas=(0.9, 0.99), epsilon=1e-8, max_preconditioner_dim=5, precondition_frequency=2, start_preconditioning_step=2)
        kw.update(_families(lib)[family])
        if family == "spectral":
            params_filter = lambda ps: [p for p in ps if p.dim() == 2]
        else:
            params_filter = list
        if extras == "adam_graft_wd":
            kw.update(grafting_config=lib.AdamPreconditionerConfig(beta2=0.99), weight_decay=0.01)
        elif extras == "momentum_beta3":
            kw.update(
                beta3=0.8, weight_decay=0.01, weight_decay_type=lib.WeightDecayType.CORRECTED,
                iterate_averaging_config=lib.shampoo_types.ClassicMomentumConfig(momentum=0.6, dampening=0.1, use_nesterov=True)
                if lib is R else lib.ClassicMomentumConfig(momentum=0.6, dampening=0.1, use_nesterov=True),
                grafting_config=lib.RMSpropPreconditionerConfig(beta2=0.95),
            )
        else:
            kw.update(
                iterate_averaging_config=lib.ScheduleFreeConfig(train_interp_coeff=0.8), weight_decay=0.02,
                weight_decay_type=lib.WeightDecayType.INDEPENDENT, grafting_config=lib.AdaGradPreconditionerConfig(),
            )
        return lambda ps: lib.DistributedShampoo(params_filter(list(ps)), **kw)

    m_ref, o_ref, l_ref = _run(build(R), steps=7)
    m_our, o_our, l_our = _run(build(ob), steps=7)
    assert l_ref == l_our
    _assert_same_params(m_ref, m_our)
    _compare_state(o_ref.state_dict()["state"], o_our.state_dict()["state"])


def _compare_state(a, b, path=""):
    if isinstance(a, dict):
        assert set(a) == set(b), (path, set(a) ^ set(b))
        for k in a:
            _compare_state(a[k], b[k], f"{path}/{k}")
    elif isinstance(a, torch.Tensor):
        assert a.shape == b.shape and a.dtype == b.dtype, path
        assert torch.equal(a, b), (path, (a.double() - b.double()).abs().max())
    else:
        assert a == b, path


@pytest.mark.skipif(not reference_available(), reason="reference not installed")
def test_checkpoints_interchange_with_reference():
    R = reference()
    kw = dict(lr=0.02, betas=(0.9, 0.99), epsilon=1e-8, max_preconditioner_dim=5, precondition_frequency=2, start_preconditioning_step=2)
    m_ref, o_ref, _ = _run(lambda p: R.DistributedShampoo(p, grafting_config=R.AdamPreconditionerConfig(), **kw), steps=4)
    m_our, o_our, _ = _run(lambda p: ob.DistributedShampoo(p, grafting_config=ob.AdamPreconditionerConfig(), **kw), steps=2)
    # the tensors of a reference checkpoint load into this optimizer (and the other way round)
    sd = o_ref.state_dict()
    mine = o_our.state_dict()
    mine["state"] = copy.deepcopy(sd["state"])
    o_our.load_state_dict(mine)
    _compare_state(o_ref.state_dict()["state"], o_our.state_dict()["state"])
    theirs = o_ref.state_dict()
    theirs["state"] = copy.deepcopy(o_our.state_dict()["state"])
    o_ref.load_state_dict(theirs)


# --------------------------------------------------------------------------------------------
# State dict, masking, validation
# --------------------------------------------------------------------------------------------
def test_state_dict_layout_and_round_trip():
    make = lambda p: ob.DistributedShampoo(
        p, lr=0.01, betas=(0.9, 0.999), max_preconditioner_dim=5, precondition_frequency=2, start_preconditioning_step=2,
        grafting_config=ob.AdamPreconditionerConfig(), iterate_averaging_config=ob.ClassicMomentumConfig(),
    )
    model, opt, _ = _run(make, steps=4)
    sd = opt.state_dict()
    first = sd["state"][0]  # Linear(10, 12).weight -> blocks of at most 5 x 5: 3 x 2 = 6 blocks
    assert {k for k in first if k.startswith("block_")} == {f"block_{i}" for i in range(6)}
    blk = first["block_0"]
    assert set(blk) == {"shampoo", "adagrad", "filtered_grad", "momentum_buffer"}
    assert set(blk["shampoo"]) == {"factor_matrices", "inv_factor_matrices"}
    assert blk["shampoo"]["factor_matrices"][0].shape == (15,)  # packed 5 x 5
    assert first["step"].item() == 4 and first["step"].device.type == "cpu"
    # continuing after a save/load into a fresh optimizer reproduces continued training bitwise
    model2 = copy.deepcopy(model)
    opt2 = make(model2.parameters())
    opt2.load_state_dict(copy.deepcopy(sd))
    for (x, y) in _batches(3, seed=9):
        for m, o in ((model, opt), (model2, opt2)):
            o.zero_grad()
            torch.nn.functional.cross_entropy(m(x), y).backward()
            o.step()
    _assert_same_params(model, model2)


def test_aliased_scalars_must_agree_on_load():
    model, opt, _ = _run(lambda p: ob.DistributedShampoo(p, max_preconditioner_dim=5), steps=2)
    sd = copy.deepcopy(opt.state_dict())
    sd["state"][1]["step"] = torch.tensor(99)
    with pytest.raises(ValueError, match="aliased across parameters"):
        opt.load_state_dict(sd)


def test_parameters_without_gradient_are_masked():
    make = lambda p: ob.DistributedShampoo(p, lr=0.01, max_preconditioner_dim=5, precondition_frequency=1, grafting_config=ob.AdaGradPreconditionerConfig())
    model, opt, _ = _run(make, steps=3, skip_grad_of=2)
    fresh = _model()
    untouched = list(fresh.parameters())[2]
    assert torch.equal(list(model.parameters())[2], untouched)
    assert not torch.equal(list(model.parameters())[0], list(fresh.parameters())[0])


@pytest.mark.parametrize(
    "kwargs,message",
    [
        (dict(lr=-1.0), "Invalid param_group[LR]=-1.0. Must be >= 0.0."),
        (dict(betas=(1.0, 1.0)), "Invalid param_group[BETAS][0]=1.0. Must be in [0.0, 1.0)."),
        (dict(betas=(0.9, 1.5)), "Must be in [0.0, 1.0]."),
        (dict(beta3=1.0), "Invalid param_group[BETA3]=1.0"),
        (dict(epsilon=0.0), "Must be > 0.0."),
        (dict(weight_decay=-0.1), "Invalid param_group[WEIGHT_DECAY]=-0.1"),
        (dict(max_preconditioner_dim=3.5), "Must be an integer or math.inf."),
        (dict(max_preconditioner_dim=0), "Must be >= 1."),
        (dict(precondition_frequency=0), "Invalid param_group[PRECONDITION_FREQUENCY]=0"),
        (dict(start_preconditioning_step=-2), "Must be >= -1."),
        (dict(start_preconditioning_step=1, precondition_frequency=5), "Must be >= param_group[PRECONDITION_FREQUENCY]=5."),
        (dict(lr=0.0, weight_decay_type=ob.WeightDecayType.CORRECTED), "Must be > 0.0 when using WeightDecayType.CORRECTED"),
    ],
)
def test_constructor_validation(kwargs, message):
    with pytest.raises(ValueError) as err:
        ob.DistributedShampoo(_model().parameters(), **kwargs)
    assert message in str(err.value)


def test_pseudo_inverse_requires_zero_epsilon_and_empty_group_is_rejected():
    cfg = ob.RootInvShampooPreconditionerConfig(
        amortized_computation_config=ob.EigenConfig(rank_deficient_stability_config=ob.PseudoInverseConfig())
    )
    with pytest.raises(ValueError, match="Must be == 0.0 when PseudoInverseConfig is used"):
        ob.DistributedShampoo(_model().parameters(), preconditioner_config=cfg)
    ob.DistributedShampoo(_model().parameters(), preconditioner_config=cfg, epsilon=0.0)
    with pytest.raises(ValueError, match="empty parameter"):
        ob.DistributedShampoo([{"params": []}])


def test_failed_refreshes_are_tolerated_then_raise(monkeypatch):
    from optimizers_b200.matrix import functions as mf

    model = _model()
    cfg = ob.RootInvShampooPreconditionerConfig(num_tolerated_failed_amortized_computations=2)
    opt = ob.DistributedShampoo(model.parameters(), max_preconditioner_dim=5, precondition_frequency=1, preconditioner_config=cfg)

    def boom(*a, **k):
        raise RuntimeError("injected")

    monkeypatch.setattr(mf, "matrix_inverse_root", boom)
    batches = _batches(4)

    def step(i):
        x, y = batches[i]
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()

    step(0)
    step(1)  # two tolerated failures: previous (identity) roots are kept
    blk = opt.state_dict()["state"][0]["block_0"]["shampoo"]["inv_factor_matrices"][0]
    assert torch.equal(blk, torch.tensor([1.0, 0, 0, 0, 0, 1, 0, 0, 0, 1, 0, 0, 1, 0, 1]))
    with pytest.raises(ValueError, match="exceeded the allowed tolerance"):
        step(2)


def test_non_finite_factor_raises_preconditioner_value_error():
    model = _model()
    opt = ob.DistributedShampoo(model.parameters(), max_preconditioner_dim=5, precondition_frequency=1)
    for p in model.parameters():
        p.grad = torch.full_like(p, float("nan"))
    with pytest.raises(ob.PreconditionerValueError, match="nan/inf values in factor matrix"):
        opt.step()


def test_exports_cover_the_reference_surface():
    names = [
        "DistributedShampoo", "ShampooPT2CompileConfig", "DistributedConfig", "SingleDeviceDistributedConfig",
        "DefaultSingleDeviceDistributedConfig", "DDPDistributedConfig", "FSDPParamAssignmentStrategy",
        "FSDPDistributedConfig", "FullyShardDistributedConfig", "HSDPDistributedConfig", "HybridShardDistributedConfig",
        "PreconditionerConfig", "BaseShampooPreconditionerConfig", "ClassicShampooPreconditionerConfig",
        "RootInvShampooPreconditionerConfig", "DefaultShampooConfig", "RootInvKLShampooPreconditionerConfig",
        "EigendecomposedShampooPreconditionerConfig", "EigendecomposedKLShampooPreconditionerConfig",
        "EigenvalueCorrectedShampooPreconditionerConfig", "DefaultEigenvalueCorrectedShampooConfig", "DefaultSOAPConfig",
        "SpectralDescentPreconditionerConfig", "SignDescentPreconditionerConfig",
        "DefaultSpectralDescentPreconditionerConfig", "DefaultSignDescentPreconditionerConfig", "SGDPreconditionerConfig",
        "AdaGradPreconditionerConfig", "RMSpropPreconditionerConfig", "AdamPreconditionerConfig",
        "RankDeficientStabilityConfig", "PerturbationConfig", "DefaultPerturbationConfig", "PseudoInverseConfig",
        "MatrixFunctionConfig", "EigendecompositionConfig", "EighEigendecompositionConfig",
        "DefaultEigendecompositionConfig", "QREigendecompositionConfig", "RootInvConfig", "EigenConfig",
        "DefaultEigenConfig", "CoupledNewtonConfig", "CoupledHigherOrderConfig", "OrthogonalizationConfig",
        "SVDOrthogonalizationConfig", "NewtonSchulzOrthogonalizationConfig", "DefaultNewtonSchulzOrthogonalizationConfig",
        "IterateAveragingConfig", "GeneralizedPrimalAveragingConfig", "ScheduleFreeConfig", "WeightDecayType",
        "compile_fsdp_parameter_metadata", "ClassicMomentumConfig", "GPAAdamW", "IterateAveragingType",
    ]
    for n in names:
        assert getattr(ob, n) is not None, n
    with pytest.raises(TypeError):
        ob.PreconditionerConfig()  # abstract


def _more_options(lib):
    R = reference()
    momentum = (lib.shampoo_types.ClassicMomentumConfig if lib is R else lib.ClassicMomentumConfig)
    return {
        "l2_without_bias_correction": dict(
            weight_decay=0.05, weight_decay_type=lib.WeightDecayType.L2, use_bias_correction=False,
            grafting_config=lib.AdamPreconditionerConfig(beta2=0.99),
        ),
        "decoupled_sgd_graft_plain_momentum": dict(
            weight_decay=0.03, weight_decay_type=lib.WeightDecayType.DECOUPLED, grafting_config=lib.SGDPreconditionerConfig(),
            iterate_averaging_config=momentum(momentum=0.9, dampening=0.0, use_nesterov=False), betas=(0.0, 0.99),
        ),
        "no_grafting_beta2_one": dict(betas=(0.9, 1.0), epsilon=1e-6),
        "rows_only": dict(
            preconditioner_config=lib.RootInvShampooPreconditionerConfig(inverse_exponent_override={2: {0: 0.25, 1: 0.0}}),
            grafting_config=lib.AdamPreconditionerConfig(beta2=0.99),
        ),
        "matrices_unpreconditioned": dict(
            preconditioner_config=lib.RootInvShampooPreconditionerConfig(inverse_exponent_override={2: 0.0}),
            grafting_config=lib.AdaGradPreconditionerConfig(),
        ),
        "eigendecomposed_columns_only": dict(
            preconditioner_config=lib.EigendecomposedShampooPreconditionerConfig(inverse_exponent_override={2: {0: 0.0, 1: 0.5}}),
            grafting_config=lib.AdamPreconditionerConfig(beta2=0.99),
        ),
        "coupled_higher_order": dict(
            preconditioner_config=lib.RootInvShampooPreconditionerConfig(
                amortized_computation_config=lib.CoupledHigherOrderConfig(rel_epsilon=1e-6, abs_epsilon=1e-10, order=3)
            ),
            grafting_config=lib.AdamPreconditionerConfig(beta2=0.99),
        ),
        "generalized_primal_averaging": dict(
            iterate_averaging_config=lib.GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.9, train_interp_coeff=0.7),
            grafting_config=lib.AdamPreconditionerConfig(beta2=0.99), weight_decay=0.01,
        ),
    }


@pytest.mark.skipif(not reference_available(), reason="reference not installed")
@pytest.mark.parametrize("name", list(_more_options(ob)))
def test_more_option_sets_match_reference_bitwise(name):
    """Option sets beyond the family x extras grid: the other weight-decay types, no bias correction,
    plain momentum, no grafting, dims switched off by an exponent of 0 (one side, or the whole
    matrix), the coupled higher-order root, and primal averaging with visits to eval mode between
    steps."""
    R = reference()

    def run(lib):
        kw = dict(lr=0.02, betas=(0.9, 0.99), epsilon=1e-8, max_preconditioner_dim=5, precondition_frequency=2, start_preconditioning_step=2)
        kw.update(_more_options(lib)[name])
        model = _model()
        opt = lib.DistributedShampoo(model.parameters(), **kw)
        opt.train()
        seen, losses = [], []
        for step, (x, y) in enumerate(_batches(7)):
            if name == "generalized_primal_averaging" and step in (3, 5):
                opt.eval()
                seen.append([p.detach().clone() for p in model.parameters()])
                opt.train()
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        seen.append([p.detach().clone() for p in model.parameters()])
        return seen, losses, opt

    seen_ref, losses_ref, o_ref = run(R)
    seen_our, losses_our, o_our = run(ob)
    assert losses_ref == losses_our
    for a_list, b_list in zip(seen_ref, seen_our, strict=True):
        for a, b in zip(a_list, b_list):
            assert torch.equal(a, b), (name, (a - b).abs().max().item())
    _compare_state(o_ref.state_dict()["state"], o_our.state_dict()["state"])


@pytest.mark.skipif(not reference_available(), reason="reference not installed")
@pytest.mark.parametrize("family", ["root_inv", "soap", "eigendecomposed_kl", "root_inv_trace_scaling_override"])
@pytest.mark.parametrize("max_dim", [3, 6, 64])
def test_convolution_weights_match_reference_bitwise(family, max_dim):
    """Order-4 weights: merged and blocked into tensors of order 1 to 4 depending on
    ``max_preconditioner_dim`` (dims merged while their product fits, then split)."""
    R = reference()

    def run(lib):
        torch.manual_seed(0)
        model = torch.nn.Sequential(
            torch.nn.Conv2d(2, 4, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(4, 3, (1, 3), padding=(0, 1)),
            torch.nn.AdaptiveAvgPool2d(1), torch.nn.Flatten(), torch.nn.Linear(3, 3),
        )
        kw = dict(lr=0.02, betas=(0.9, 0.99), epsilon=1e-8, max_preconditioner_dim=max_dim, precondition_frequency=2,
                  start_preconditioning_step=2, grafting_config=lib.AdamPreconditionerConfig(beta2=0.99), weight_decay=0.01)
        kw.update(_families(lib)[family])
        opt = lib.DistributedShampoo(model.parameters(), **kw)
        g = torch.Generator().manual_seed(3)
        losses = []
        for _ in range(6):
            x, y = torch.randn(8, 2, 5, 5, generator=g), torch.randint(0, 3, (8,), generator=g)
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        return model, opt, losses

    m_ref, o_ref, l_ref = run(R)
    m_our, o_our, l_our = run(ob)
    assert l_ref == l_our
    _assert_same_params(m_ref, m_our)
    _compare_state(o_ref.state_dict()["state"], o_our.state_dict()["state"])


@pytest.mark.skipif(not reference_available(), reason="reference not installed")
@pytest.mark.parametrize("scenario", ["lr_schedule_corrected_wd", "lr_schedule_schedule_free", "lr_schedule_primal_averaging", "two_groups_and_a_frozen_parameter"])
def test_schedules_and_parameter_groups_match_reference_bitwise(scenario):
    """The learning rate changes every step (warm-up, then decay), which feeds the corrected weight
    decay, the Schedule-Free weights and the primal-averaging coefficients; and two parameter groups
    with different preconditioners, one of them holding a frozen parameter."""
    R = reference()

    def run(lib):
        model = _model()
        momentum = lib.shampoo_types.ClassicMomentumConfig if lib is R else lib.ClassicMomentumConfig
        kw = dict(lr=0.02, betas=(0.9, 0.99), epsilon=1e-8, max_preconditioner_dim=5, precondition_frequency=2, start_preconditioning_step=2,
                  grafting_config=lib.AdamPreconditionerConfig(beta2=0.99))
        params = list(model.parameters())
        if scenario == "lr_schedule_corrected_wd":
            kw.update(weight_decay=0.05, weight_decay_type=lib.WeightDecayType.CORRECTED,
                      iterate_averaging_config=momentum(momentum=0.8, dampening=0.0, use_nesterov=True))
            groups = params
        elif scenario == "lr_schedule_schedule_free":
            kw.update(iterate_averaging_config=lib.ScheduleFreeConfig(train_interp_coeff=0.9), weight_decay=0.01)
            groups = params
        elif scenario == "lr_schedule_primal_averaging":
            kw.update(iterate_averaging_config=lib.GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.95, train_interp_coeff=0.6))
            groups = params
        else:
            params[1].requires_grad_(False)
            groups = [
                dict(params=params[:2], lr=0.01, preconditioner_config=lib.DefaultSOAPConfig),
                dict(params=params[2:], weight_decay=0.02, max_preconditioner_dim=4),
            ]
        opt = lib.DistributedShampoo(groups, **kw)
        opt.train()
        losses = []
        for step, (x, y) in enumerate(_batches(8)):
            if scenario.startswith("lr_schedule"):
                for group in opt.param_groups:
                    group["lr"] = 0.02 * min(1.0, (step + 1) / 3) * (0.8 ** max(0, step - 3))
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        opt.eval()
        return model, opt, losses

    m_ref, o_ref, l_ref = run(R)
    m_our, o_our, l_our = run(ob)
    assert l_ref == l_our
    _assert_same_params(m_ref, m_our)
    _compare_state(o_ref.state_dict()["state"], o_our.state_dict()["state"])


def test_cpu_mlp_configuration_of_the_baseline_matches_reference_bitwise():
    """The CPU configuration that serves as the oracle: MLP 784-512-10, batch 64, 100 steps, lr 1e-3,
    betas (0.9, 0.999), epsilon 1e-12, blocks of 256, refresh every 10 steps from step 10, Adam
    grafting, root-inverse Shampoo by eigendecomposition.  Losses and parameters of all 100 steps
    are identical to the reference's (``distributed_shampoo/distributed_shampoo.py``)."""
    from ref_oracle import reference, reference_available

    if not reference_available():
        pytest.skip("reference not installed")

    def run(lib):
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, 512), torch.nn.ReLU(), torch.nn.Linear(512, 10))
        opt = lib.DistributedShampoo(
            model.parameters(), lr=1e-3, betas=(0.9, 0.999), epsilon=1e-12, max_preconditioner_dim=256,
            precondition_frequency=10, start_preconditioning_step=10,
            grafting_config=lib.AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8),
            preconditioner_config=lib.DefaultShampooConfig,
        )
        g = torch.Generator().manual_seed(1)
        losses = []
        for _ in range(100):
            x, y = torch.randn(64, 1, 28, 28, generator=g), torch.randint(0, 10, (64,), generator=g)
            opt.zero_grad()
            loss = torch.nn.functional.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        return losses, [p.detach().clone() for p in model.parameters()]

    their_losses, their_params = run(reference())
    my_losses, my_params = run(ob)
    assert their_losses == my_losses
    assert all(torch.equal(a, b) for a, b in zip(their_params, my_params, strict=True))
