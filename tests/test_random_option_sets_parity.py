"""Random option sets against the installed reference, bit for bit.

Each seed draws a preconditioner family with its matrix-function configuration, packing,
per-order exponent overrides, trace scaling, ignored basis changes, a grafting method, betas,
beta3, epsilon, weight decay and its type, an iterate-averaging scheme, bias correction, block
size, refresh frequency and start step, and one of two small models (an MLP, or a convolution in
front of a linear layer).  Both libraries then either refuse the combination with the same
exception, or fail in the same step with the same kind of error, or train for seven steps with a
visit to ``eval()`` in between and end with identical parameters
(``distributed_shampoo/distributed_shampoo.py`` and ``preconditioner/*.py`` in the reference).
"""

import logging
import math
import random

import pytest
import torch

import optimizers_b200 as ob
from ref_oracle import reference, reference_available

pytestmark = pytest.mark.skipif(not reference_available(), reason="the reference is not installed under baseline/_ref")


def _get(lib, name):
    # the reference does not re-export every configuration class from its package root
    return getattr(lib, name) if hasattr(lib, name) else getattr(lib.shampoo_types, name)


def _options(lib, rng):
    """One option set, built from ``lib``'s classes; ``rng`` is consumed the same way for both."""
    family = rng.choice([
        "root_inv", "root_inv_newton", "root_inv_higher_order", "eigendecomposed", "eigendecomposed_qr",
        "eigenvalue_corrected", "eigenvalue_corrected_qr", "kl_root_inv", "kl_eigendecomposed", "sign", "spectral",
    ])
    packing = rng.random() < 0.5
    override = rng.choice([{}, {2: 0.25}, {2: {0: 0.5, 1: 0.0}}, {1: 0.0}, {1: 0.5, 2: {0: 0.0}}])
    kw = {}
    if family.startswith("root_inv") or family == "kl_root_inv":
        cls = lib.RootInvKLShampooPreconditionerConfig if family == "kl_root_inv" else lib.RootInvShampooPreconditionerConfig
        computation = {
            "root_inv": lib.EigenConfig(), "kl_root_inv": lib.EigenConfig(), "root_inv_newton": lib.CoupledNewtonConfig(),
            "root_inv_higher_order": lib.CoupledHigherOrderConfig(rel_epsilon=1e-6, abs_epsilon=1e-10, order=rng.choice([2, 3])),
        }[family]
        kw["preconditioner_config"] = cls(
            amortized_computation_config=computation, use_symmetric_packing=packing, inverse_exponent_override=override,
            use_trace_scaling=rng.random() < 0.3, num_tolerated_failed_amortized_computations=3,
        )
    elif family in ("eigendecomposed", "eigendecomposed_qr", "kl_eigendecomposed"):
        cls = lib.EigendecomposedKLShampooPreconditionerConfig if family == "kl_eigendecomposed" else lib.EigendecomposedShampooPreconditionerConfig
        computation = (
            lib.QREigendecompositionConfig(max_iterations=rng.choice([1, 2])) if family == "eigendecomposed_qr"
            else lib.EighEigendecompositionConfig()
        )
        kw["preconditioner_config"] = cls(
            amortized_computation_config=computation, use_symmetric_packing=packing, inverse_exponent_override=override
        )
    elif family.startswith("eigenvalue_corrected"):
        computation = (
            lib.QREigendecompositionConfig(max_iterations=rng.choice([1, 3])) if family == "eigenvalue_corrected_qr"
            else lib.EighEigendecompositionConfig()
        )
        kw["preconditioner_config"] = lib.EigenvalueCorrectedShampooPreconditionerConfig(
            amortized_computation_config=computation, use_symmetric_packing=packing,
            inverse_exponent_override=rng.choice([{}, {2: 0.25}, {1: 1.0, 2: 0.5}]),
            ignored_basis_change_dims=rng.choice([{}, {2: [0]}, {2: [1]}]),
        )
    elif family == "sign":
        kw["preconditioner_config"] = lib.DefaultSignDescentPreconditionerConfig
    else:
        kw["preconditioner_config"] = lib.DefaultSpectralDescentPreconditionerConfig
        kw["max_preconditioner_dim"] = math.inf
        kw["distributed_config"] = lib.SingleDeviceDistributedConfig(target_parameter_dimensionality=2)
    grafting = rng.choice(["none", "sgd", "adagrad", "rmsprop", "adam"])
    if family != "sign":
        kw["grafting_config"] = {
            "none": None, "sgd": lib.SGDPreconditionerConfig(), "adagrad": lib.AdaGradPreconditionerConfig(epsilon=1e-8),
            "rmsprop": lib.RMSpropPreconditionerConfig(beta2=0.95), "adam": lib.AdamPreconditionerConfig(beta2=0.99),
        }[grafting]
    kw["betas"] = (rng.choice([0.0, 0.5, 0.9]), rng.choice([1.0, 0.99, 0.9]))
    if rng.random() < 0.4 and kw["betas"][0] > 0:
        kw["beta3"] = rng.choice([0.0, 0.7])
    kw["epsilon"] = rng.choice([1e-12, 1e-6, 1e-3])
    kw["weight_decay"] = rng.choice([0.0, 1e-2])
    kw["weight_decay_type"] = rng.choice(list(lib.WeightDecayType))
    momentum = _get(lib, "ClassicMomentumConfig")
    kw["iterate_averaging_config"] = {
        "none": None, "momentum": momentum(momentum=0.5, dampening=0.1), "nesterov": momentum(momentum=0.9, use_nesterov=True),
        "primal_averaging": lib.GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.9, train_interp_coeff=0.7),
        "schedule_free": lib.ScheduleFreeConfig(train_interp_coeff=0.9),
    }[rng.choice(["none", "momentum", "nesterov", "primal_averaging", "schedule_free"])]
    kw["use_bias_correction"] = rng.random() < 0.7
    kw.setdefault("max_preconditioner_dim", rng.choice([4, 7, 16, math.inf]))
    kw["precondition_frequency"] = rng.choice([1, 2, 3])
    start = rng.choice([-1, 3, 4])
    kw["start_preconditioning_step"] = start if start >= kw["precondition_frequency"] else -1
    kw["lr"] = rng.choice([1e-2, 1e-1])
    return family, kw


def _strip(text):
    text = text.replace("distributed_shampoo.", "").replace("optimizers_b200.", "")
    if "Encountered nan or inf values in" in text:
        # the reference prints the literal word "name" for the quantity (a formatting slip in
        # preconditioner/shampoo_preconditioner_list.py:412-417); this library names the quantity
        return "non-finite result of a matrix computation"
    return text[:150]


def _outcome(lib, seed):
    rng = random.Random(seed)
    family, kw = _options(lib, rng)
    torch.manual_seed(seed)
    if rng.random() < 0.3 and family != "spectral":
        model = torch.nn.Sequential(torch.nn.Conv2d(2, 4, 3), torch.nn.Flatten(), torch.nn.Linear(4 * 4 * 4, 3))
        shape = (8, 2, 6, 6)
    else:
        model = torch.nn.Sequential(torch.nn.Linear(9, 12), torch.nn.Tanh(), torch.nn.Linear(12, 3, bias=False))
        shape = (8, 9)
    try:
        opt = lib.DistributedShampoo(model.parameters(), **kw)
    except Exception as err:  # noqa: BLE001 - the kind and the text are what is compared
        return f"constructor: {type(err).__name__}: {_strip(str(err))}", None
    g = torch.Generator().manual_seed(seed + 1)
    opt.train()
    try:
        for step in range(7):
            x, y = torch.randn(*shape, generator=g), torch.randint(0, 3, (8,), generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
            if step == 4:
                opt.eval()
                opt.train()
        opt.eval()
    except Exception as err:  # noqa: BLE001
        return f"step: {type(err).__name__}: {_strip(str(err))}", None
    return "trained", [p.detach().clone() for p in model.parameters()]


@pytest.mark.parametrize("first_seed", [0, 12, 24, 36])
def test_random_option_sets_match_reference_bitwise(first_seed):
    logging.disable(logging.WARNING)  # both libraries log every tolerated failure
    try:
        trained = 0
        for seed in range(first_seed, first_seed + 12):
            theirs, their_params = _outcome(reference(), seed)
            mine, my_params = _outcome(ob, seed)
            assert theirs == mine, (seed, theirs, mine)
            if their_params is not None:
                trained += 1
                for a, b in zip(their_params, my_params, strict=True):
                    assert torch.equal(a, b), (seed, (a - b).abs().max().item())
        assert trained >= 6
    finally:
        logging.disable(logging.NOTSET)


def _same_tree(a, b, path="state"):
    """None when two state trees agree (keys, tensor shapes / dtypes / values, other leaves by
    repr), else a description of the first difference."""
    if isinstance(a, dict):
        if set(map(str, a)) != set(map(str, b)):
            return f"{path}: keys differ"
        for key in a:
            found = _same_tree(a[key], b[key], f"{path}/{key}")
            if found:
                return found
        return None
    if isinstance(a, torch.Tensor):
        same = a.shape == b.shape and a.dtype == b.dtype and torch.equal(a, b)
        return None if same else f"{path}: tensor differs"
    return None if _strip(repr(a)) == _strip(repr(b)) else f"{path}: {a!r} against {b!r}"


def test_checkpoints_of_random_option_sets_interchange_with_the_reference():
    """For each option set: after four steps the two ``state_dict()["state"]`` trees are identical;
    a fresh reference optimizer resumed from this library's checkpoint, and a fresh optimizer of
    this library resumed from the reference's, continue exactly like the uninterrupted runs."""
    import copy

    logging.disable(logging.WARNING)

    def make(lib, seed):
        _, kw = _options(lib, random.Random(seed))
        torch.manual_seed(seed)
        model = torch.nn.Sequential(torch.nn.Linear(9, 12), torch.nn.Tanh(), torch.nn.Linear(12, 3, bias=False))
        return model, lib.DistributedShampoo(model.parameters(), **kw)

    def train(model, opt, data_seed, steps):
        g = torch.Generator().manual_seed(data_seed)
        opt.train()
        for _ in range(steps):
            x, y = torch.randn(8, 9, generator=g), torch.randint(0, 3, (8,), generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()

    checked = 0
    try:
        for seed in range(100, 124):
            try:
                (their_model, theirs), (my_model, mine) = make(reference(), seed), make(ob, seed)
                train(their_model, theirs, seed, 4)
                train(my_model, mine, seed, 4)
            except Exception:  # noqa: BLE001 - refused or failing option sets are the other tests' topic
                continue
            their_state, my_state = theirs.state_dict(), mine.state_dict()
            assert _same_tree(their_state["state"], my_state["state"]) is None, seed
            (their_model2, theirs2), (my_model2, mine2) = make(reference(), seed), make(ob, seed)
            their_model2.load_state_dict(my_model.state_dict())
            my_model2.load_state_dict(their_model.state_dict())
            for fresh, source in ((theirs2, my_state), (mine2, their_state)):
                checkpoint = fresh.state_dict()
                checkpoint["state"] = copy.deepcopy(source["state"])
                fresh.load_state_dict(checkpoint)
            try:
                runs = ((their_model, theirs), (my_model, mine), (their_model2, theirs2), (my_model2, mine2))
                for model, opt in runs:
                    train(model, opt, seed + 7, 3)
            except Exception:  # noqa: BLE001
                continue
            for model, _ in runs[1:]:
                for a, b in zip(their_model.parameters(), model.parameters(), strict=True):
                    assert torch.equal(a, b), seed
            checked += 1
        assert checked >= 12
    finally:
        logging.disable(logging.NOTSET)
