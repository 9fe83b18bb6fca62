"""GPAAdamW on CPU: validation, modes, AdamW equivalence, averaging coefficient, checkpoint."""

import copy

import pytest
import torch

from optimizers_b200.gpa_adamw import GPAAdamW, IterateAveragingType


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh(), torch.nn.Linear(8, 2))


def _train(opt_fn, steps=8):
    model = _model()
    opt = opt_fn(model.parameters())
    if hasattr(opt, "train"):
        opt.train()
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        x, y = torch.randn(16, 6, generator=g), torch.randn(16, 2, generator=g)
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(x), y).backward()
        opt.step()
    return model, opt


@pytest.mark.parametrize(
    "kwargs,message",
    [
        (dict(lr=-1), "Invalid learning rate"), (dict(eps=-1), "Invalid epsilon"), (dict(beta1=1.0), "Invalid beta1"),
        (dict(beta2=-0.1), "Invalid beta2"), (dict(weight_decay=-1), "Invalid weight_decay"),
        (dict(iterate_averaging_type="gpa"), "must be an IterateAveragingType"), (dict(train_interp_coeff=0.0), "train_interp_coeff"),
        (dict(eval_interp_coeff=1.5), "eval_interp_coeff"), (dict(weight_pow_coeff=-1), "weight_pow_coeff"),
        (dict(weight_lr_power=-1), "weight_lr_power"),
    ],
)
def test_validation(kwargs, message):
    with pytest.raises(ValueError, match=message):
        GPAAdamW(_model().parameters(), **kwargs)


def test_starts_in_eval_mode_and_step_requires_train():
    model = _model()
    opt = GPAAdamW(model.parameters(), lr=0.01)
    for p in model.parameters():
        p.grad = torch.ones_like(p)
    with pytest.raises(RuntimeError, match="not in train mode"):
        opt.step()
    opt.train()
    opt.step()
    first = next(iter(model.parameters()))
    assert set(opt.state[first]) == {"train_mode", "lr_max", "weight_sum", "step", "z", "exp_avg", "exp_avg_sq"}
    second = list(model.parameters())[1]
    assert set(opt.state[second]) == {"z", "exp_avg", "exp_avg_sq"}


def test_mu_x_zero_is_adamw():
    m_ref, _ = _train(lambda p: torch.optim.AdamW(p, lr=0.01, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1))
    m_gpa, opt = _train(lambda p: GPAAdamW(p, lr=0.01, eps=1e-8, weight_decay=0.1, eval_interp_coeff=0.0, train_interp_coeff=1.0))
    for a, b in zip(m_ref.parameters(), m_gpa.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


def test_mode_round_trip_and_checkpoint():
    model, opt = _train(lambda p: GPAAdamW(p, lr=0.01, weight_decay=0.01))
    y = [p.detach().clone() for p in model.parameters()]
    opt.eval()
    assert any(not torch.equal(a, b) for a, b in zip(y, model.parameters()))
    opt.train()
    for a, b in zip(y, model.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    sd = copy.deepcopy(opt.state_dict())
    model2 = copy.deepcopy(model)
    opt2 = GPAAdamW(model2.parameters(), lr=0.01, weight_decay=0.01)
    opt2.load_state_dict(sd)
    for m, o in ((model, opt), (model2, opt2)):
        for p in m.parameters():
            p.grad = torch.full_like(p, 0.5)
        o.step()
    for a, b in zip(model.parameters(), model2.parameters()):
        assert torch.equal(a, b)


def test_avg_coeff():
    ws = torch.tensor(0.0)
    assert GPAAdamW.compute_avg_coeff(IterateAveragingType.GPA, 0.9, 3, 0.0, 1.0, 2.0, ws) == pytest.approx(0.1)
    c1 = GPAAdamW.compute_avg_coeff(IterateAveragingType.SCHEDULE_FREE, 0.0, 1, 0.0, 0.5, 2.0, ws)
    c2 = GPAAdamW.compute_avg_coeff(IterateAveragingType.SCHEDULE_FREE, 0.0, 2, 0.0, 0.5, 2.0, ws)
    assert float(c1) == pytest.approx(1.0) and float(c2) == pytest.approx(0.5) and float(ws) == pytest.approx(0.5)


def test_schedule_free_converges_on_quadratic():
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.tensor([3.0, -2.0]))
    opt = GPAAdamW([w], lr=0.1, iterate_averaging_type=IterateAveragingType.SCHEDULE_FREE, train_interp_coeff=0.9)
    opt.train()
    for _ in range(300):
        opt.zero_grad()
        (w**2).sum().backward()
        opt.step()
    opt.eval()
    assert w.abs().max() < 0.3  # the average of the iterates lags behind the last iterate
