"""The public surface against the installed reference, name by name.

Every name the reference exports from ``distributed_shampoo/__init__.py`` must exist here with the
same kind: dataclasses with the same fields, defaults, keyword-only flags and base-class chain,
enums with the same members in the same order, ready-made configurations with the same contents,
and optimizer constructors with the same parameters and defaults (``distributed_shampoo.py`` and
``gpa/gpa_adamw.py`` in the reference).  A user's keyword arguments and ``isinstance`` checks then
carry over unchanged.
"""

import dataclasses
import enum
import inspect

import pytest

import optimizers_b200 as ob
from ref_oracle import reference, reference_available

pytestmark = pytest.mark.skipif(not reference_available(), reason="the reference is not installed under baseline/_ref")


def _norm(value) -> str:
    """repr with the package prefixes and object addresses taken out."""
    return repr(value).replace("distributed_shampoo.", "").replace("optimizers_b200.", "").split(" at 0x")[0]


def _default(field):
    if field.default is not dataclasses.MISSING:
        return field.default
    if field.default_factory is not dataclasses.MISSING:
        return field.default_factory()
    return "<required>"


def _names():
    return sorted(reference().__all__)


def test_every_exported_name_exists():
    missing = [name for name in _names() if not hasattr(ob, name)]
    assert not missing, missing
    assert len(_names()) >= 50


def test_dataclasses_have_the_same_fields_defaults_and_bases():
    ref = reference()
    checked = 0
    for name in _names():
        theirs, mine = getattr(ref, name), getattr(ob, name)
        if not (isinstance(theirs, type) and dataclasses.is_dataclass(theirs)):
            continue
        assert dataclasses.is_dataclass(mine), name
        their_fields = {f.name: f for f in dataclasses.fields(theirs)}
        my_fields = {f.name: f for f in dataclasses.fields(mine)}
        assert list(their_fields) == list(my_fields), (name, set(their_fields) ^ set(my_fields))
        for key, field in their_fields.items():
            assert _norm(_default(field)) == _norm(_default(my_fields[key])), (name, key)
            assert field.kw_only == my_fields[key].kw_only, (name, key)
            assert field.init == my_fields[key].init, (name, key)
        # the chain of bases, by name: isinstance(config, SomeBase) gives the same answer
        their_bases = [c.__name__ for c in theirs.__mro__ if c.__module__.startswith("distributed_shampoo")]
        my_bases = [c.__name__ for c in mine.__mro__ if c.__module__.startswith("optimizers_b200")]
        assert their_bases == my_bases, name
        assert inspect.isabstract(theirs) == inspect.isabstract(mine), name
        checked += 1
    assert checked >= 30


def test_enums_and_ready_made_configurations():
    ref = reference()
    enums = instances = 0
    for name in _names():
        theirs, mine = getattr(ref, name), getattr(ob, name)
        if isinstance(theirs, type) and issubclass(theirs, enum.Enum):
            assert [(e.name, _norm(e.value)) for e in theirs] == [(e.name, _norm(e.value)) for e in mine], name
            enums += 1
        elif dataclasses.is_dataclass(theirs) and not isinstance(theirs, type):
            assert _norm(theirs) == _norm(mine), name
            instances += 1
    assert enums >= 2 and instances >= 5


def _same_parameters(theirs, mine, extra=()):
    their_sig, my_sig = inspect.signature(theirs), inspect.signature(mine)
    for key, param in their_sig.parameters.items():
        assert key in my_sig.parameters, key
        other = my_sig.parameters[key]
        assert param.kind == other.kind, key
        assert _norm(param.default) == _norm(other.default), key
    assert [k for k in my_sig.parameters if k not in their_sig.parameters] == list(extra)
    shared = [k for k in my_sig.parameters if k in their_sig.parameters]
    assert shared == list(their_sig.parameters), "positional order differs"


def test_optimizer_constructors_take_the_same_arguments():
    ref = reference()
    # this framework adds one keyword, for the choice between the CUDA engine and the torch step
    _same_parameters(ref.DistributedShampoo.__init__, ob.DistributedShampoo.__init__, extra=("native_runtime_config",))
    for method in ("step", "train", "eval", "state_dict", "load_state_dict", "zero_grad", "add_param_group"):
        assert hasattr(ob.DistributedShampoo, method), method
        _same_parameters(getattr(ref.DistributedShampoo, method), getattr(ob.DistributedShampoo, method))


def test_gpa_adamw_takes_the_same_arguments():
    import importlib

    reference()  # puts the reference on the path
    theirs = importlib.import_module("gpa.gpa_adamw").GPAAdamW
    their_sig, my_sig = inspect.signature(theirs.__init__), inspect.signature(ob.GPAAdamW.__init__)
    for key, param in their_sig.parameters.items():
        assert key in my_sig.parameters, key
        assert _norm(param.default) == _norm(my_sig.parameters[key].default), key
    for method in ("step", "train", "eval"):
        assert hasattr(ob.GPAAdamW, method)


def _constructor_cases(lib):
    """Keyword arguments the constructor must accept or refuse, built from ``lib``'s own classes
    (hyperparameter checks of ``distributed_shampoo.py`` in the reference)."""
    import math

    pseudo = lib.RootInvShampooPreconditionerConfig(
        amortized_computation_config=lib.EigenConfig(rank_deficient_stability_config=lib.PseudoInverseConfig())
    )
    return {
        "negative lr": dict(lr=-0.1),
        "beta1 below range": dict(betas=(-0.1, 1.0)),
        "beta1 of one": dict(betas=(1.0, 1.0)),
        "beta2 of zero": dict(betas=(0.1, 0.0)),
        "beta2 above range": dict(betas=(0.1, 1.1)),
        "beta3 below range": dict(beta3=-0.1),
        "beta3 of one": dict(beta3=1.0),
        "epsilon of zero": dict(epsilon=0.0),
        "negative epsilon": dict(epsilon=-1.0),
        "negative weight decay": dict(weight_decay=-0.1),
        "block size of zero": dict(max_preconditioner_dim=0),
        "fractional block size": dict(max_preconditioner_dim=1.5),
        "unbounded block size": dict(max_preconditioner_dim=math.inf),
        "frequency of zero": dict(precondition_frequency=0),
        "start below -1": dict(start_preconditioning_step=-2),
        "start before the first refresh": dict(precondition_frequency=10, start_preconditioning_step=5),
        "pseudo-inverse with a ridge": dict(epsilon=1e-12, preconditioner_config=pseudo),
        "pseudo-inverse without a ridge": dict(epsilon=0.0, preconditioner_config=pseudo),
        "sign descent with grafting": dict(
            preconditioner_config=lib.DefaultSignDescentPreconditionerConfig,
            grafting_config=lib.AdaGradPreconditionerConfig(epsilon=1e-8),
        ),
        "a string as distributed_config": dict(distributed_config="ddp"),
        "a string as iterate_averaging_config": dict(iterate_averaging_config="momentum"),
        "a string as preconditioner_config": dict(preconditioner_config="shampoo"),
    }


@pytest.mark.parametrize("case", sorted(_constructor_cases(ob)))
def test_constructor_refuses_and_accepts_what_the_reference_does(case):
    import torch

    outcomes = []
    for lib in (reference(), ob):
        model = torch.nn.Linear(4, 3)
        try:
            lib.DistributedShampoo(model.parameters(), **_constructor_cases(lib)[case])
            outcomes.append("accepted")
        except Exception as err:  # noqa: BLE001 - the kind and the text are what is compared
            outcomes.append(f"{type(err).__name__}: {_norm(str(err))}")
    assert outcomes[0] == outcomes[1]


_FIELD_VALUES = [
    -1, 0, 0.0, 0.5, 1, 1.0, 1.5, 2, -0.5, float("inf"), True, None, "x", {2: 0.5}, {2: {0: 0.25}}, {-1: 1.0},
    {2: [0]}, {2: [0, 0]}, {2: [5]}, (1.0, 2.0, 3.0),
]


def test_every_config_field_validates_like_the_reference():
    """Each constructible configuration class, each of its fields, a grid of values of several
    types: both libraries accept the same ones (and build equal objects) and refuse the others
    with the same exception type and text (``__post_init__`` checks of ``shampoo_types.py`` and
    ``preconditioner/matrix_functions_types.py`` in the reference)."""
    ref = reference()
    combinations, different = 0, []
    for name in _names():
        theirs, mine = getattr(ref, name), getattr(ob, name)
        if not (isinstance(theirs, type) and dataclasses.is_dataclass(theirs)) or inspect.isabstract(theirs):
            continue
        for field in dataclasses.fields(theirs):
            if not field.init:
                continue
            for value in _FIELD_VALUES:
                outcome = []
                for cls in (theirs, mine):
                    try:
                        outcome.append("accepted: " + _norm(cls(**{field.name: value})))
                    except Exception as err:  # noqa: BLE001 - the kind and the text are what is compared
                        outcome.append(f"{type(err).__name__}: {_norm(str(err))}")
                combinations += 1
                if outcome[0] != outcome[1]:
                    different.append((name, field.name, value, outcome))
    assert combinations > 2000
    assert not different, different[:5]
