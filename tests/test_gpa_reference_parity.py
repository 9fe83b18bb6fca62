"""GPAAdamW against the reference's own ``gpa.gpa_adamw.GPAAdamW`` on the CPU, bit for bit.

The reference's ``gpa`` package is not part of its wheel; the tests run where it has been copied
beside the installed reference (``baseline/_ref/gpa``) and skip elsewhere.  Parameters are compared
after every mode switch, and the optimizer state (``z``, ``exp_avg_sq``, the scalars) at the end.
"""

import importlib
import os
import sys

import pytest
import torch

from optimizers_b200.gpa_adamw import GPAAdamW, IterateAveragingType
from ref_oracle import REF_DIR

needs_reference_gpa = pytest.mark.skipif(
    not os.path.isdir(os.path.join(REF_DIR, "gpa")), reason="the reference's gpa package is not beside baseline/_ref"
)


def _reference():
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module("gpa.gpa_adamw"), importlib.import_module("gpa.gpa_types")


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh(), torch.nn.Linear(8, 2))


def _run(make_optimizer, schedule):
    """Train with a fixed data stream; ``schedule`` lists, per step, whether to visit eval mode
    (and come back) before the step.  Returns the parameters seen in every mode, and the optimizer."""
    model = _model()
    opt = make_optimizer(model.parameters())
    opt.train()
    g = torch.Generator().manual_seed(1)
    seen = []
    for visit_eval in schedule:
        if visit_eval:
            opt.eval()
            seen.append([p.detach().clone() for p in model.parameters()])
            opt.train()
            seen.append([p.detach().clone() for p in model.parameters()])
        x, y = torch.randn(16, 6, generator=g), torch.randn(16, 2, generator=g)
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(x), y).backward()
        opt.step()
        seen.append([p.detach().clone() for p in model.parameters()])
    opt.eval()
    seen.append([p.detach().clone() for p in model.parameters()])
    return seen, opt


_CASES = {
    "gpa_defaults": dict(lr=0.01),
    "gpa_weight_decay": dict(lr=0.01, weight_decay=0.1, train_interp_coeff=0.5, eval_interp_coeff=0.9),
    "gpa_weight_decay_on_y": dict(lr=0.02, weight_decay=0.05, use_wd_on_y=True, beta1=0.8, beta2=0.99, eps=1e-6),
    "schedule_free": dict(lr=0.01, schedule_free=True, weight_decay=0.01),
    "schedule_free_weighted": dict(lr=0.01, schedule_free=True, weight_pow_coeff=1.0, weight_lr_power=1.0),
    "tensor_lr": dict(lr=torch.tensor(0.01)),
}


@needs_reference_gpa
@pytest.mark.parametrize("name", sorted(_CASES))
def test_gpa_adamw_matches_the_reference_bitwise(name):
    ref_module, ref_types = _reference()
    kwargs = dict(_CASES[name])
    schedule_free = kwargs.pop("schedule_free", False)
    ours = dict(kwargs, use_native_kernels=False)
    theirs = dict(kwargs)
    if schedule_free:
        ours["iterate_averaging_type"] = IterateAveragingType.SCHEDULE_FREE
        theirs["iterate_averaging_type"] = ref_types.IterateAveragingType.SCHEDULE_FREE
    schedule = [False, False, True, False, True, False, False, True]
    want, ref_opt = _run(lambda p: ref_module.GPAAdamW(p, **theirs), schedule)
    got, our_opt = _run(lambda p: GPAAdamW(p, **ours), schedule)
    assert len(want) == len(got)
    for step, (a_list, b_list) in enumerate(zip(want, got)):
        for a, b in zip(a_list, b_list):
            assert torch.equal(a, b), (name, step, (a - b).abs().max().item())
    ref_state, our_state = ref_opt.state_dict()["state"], our_opt.state_dict()["state"]
    assert ref_state.keys() == our_state.keys()
    for index in ref_state:
        assert ref_state[index].keys() == our_state[index].keys(), (ref_state[index].keys(), our_state[index].keys())
        for key, value in ref_state[index].items():
            other = our_state[index][key]
            if isinstance(value, torch.Tensor):
                assert torch.equal(value, other), (name, index, key)
            else:
                assert value == other, (name, index, key)
    ref_groups, our_groups = ref_opt.state_dict()["param_groups"], our_opt.state_dict()["param_groups"]
    for rg, og in zip(ref_groups, our_groups):
        for key, value in rg.items():
            if key == "iterate_averaging_type":
                assert value.name == og[key].name
            elif isinstance(value, torch.Tensor):
                assert torch.equal(value, og[key]), key
            else:
                assert value == og[key], (key, value, og[key])


def _random_run(cls, averaging_types, seed):
    """Hyperparameters, mode visits and learning-rate cuts drawn from ``seed``; the parameters seen
    in eval mode along the way and at the end."""
    import random

    rng = random.Random(seed)
    kw = dict(
        lr=rng.choice([1e-3, 1e-2, 0.1, 1.0]), eps=rng.choice([1e-8, 1e-6]), beta1=rng.choice([0.0, 0.5, 0.9]),
        beta2=rng.choice([0.9, 0.999]), weight_decay=rng.choice([0, 1e-2, 0.1]), use_wd_on_y=rng.random() < 0.5,
        iterate_averaging_type=rng.choice(list(averaging_types)), train_interp_coeff=rng.choice([0.7, 0.9, 1.0]),
        eval_interp_coeff=rng.choice([0.0, 0.9, 0.9967]), weight_pow_coeff=rng.choice([0.0, 1.0]),
        weight_lr_power=rng.choice([0, 2]),
    )
    if rng.random() < 0.3:
        kw["lr"] = torch.tensor(kw["lr"])
    torch.manual_seed(seed)
    model = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh(), torch.nn.Linear(8, 2))
    opt = cls(model.parameters(), **kw)
    opt.train()
    g = torch.Generator().manual_seed(seed + 1)
    seen = []
    for _ in range(9):
        if rng.random() < 0.3:
            opt.eval()
            seen.append([p.detach().clone() for p in model.parameters()])
            opt.train()
        if rng.random() < 0.2:
            for group in opt.param_groups:
                group["lr"] = group["lr"] * 0.5
        x, y = torch.randn(16, 6, generator=g), torch.randn(16, 2, generator=g)
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(x), y).backward()
        opt.step()
    opt.eval()
    seen.append([p.detach().clone() for p in model.parameters()])
    return seen


@needs_reference_gpa
def test_random_hyperparameters_and_mode_visits_match_reference_bitwise():
    their_module, their_types = _reference()
    for seed in range(40):
        want = _random_run(their_module.GPAAdamW, their_types.IterateAveragingType, seed)
        got = _random_run(GPAAdamW, IterateAveragingType, seed)
        assert len(want) == len(got)
        for a_list, b_list in zip(want, got):
            for a, b in zip(a_list, b_list, strict=True):
                assert torch.equal(a, b), (seed, (a - b).abs().max().item())
