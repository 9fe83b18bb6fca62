"""The divide-and-conquer eigensolver through its plain-tensor backend (runs on CPU): the same
driver, split-point, retry and closing logic that the sm_100a backend executes."""

import pytest
import torch

from optimizers_b200.matrix.eigh_dc import SIGN_SCHEDULE, TorchBackend, eigh_divide_and_conquer


def _orth(d, gen):
    q, _ = torch.linalg.qr(torch.randn(d, d, dtype=torch.float64, generator=gen))
    return q


def _matrix(kind, d, gen):
    if kind == "lowrank":
        G = torch.randn(d, d // 3, dtype=torch.float64, generator=gen)
        return G @ G.T / d
    lam = {
        "power": 1.0 / torch.arange(1, d + 1, dtype=torch.float64) ** 2,
        "uniform": torch.rand(d, dtype=torch.float64, generator=gen),
        "clustered": torch.cat([torch.ones(d // 2), torch.full((d - d // 2,), 1e-3)]).double(),
        "scalar": torch.full((d,), 0.37, dtype=torch.float64),
    }[kind]
    q = _orth(d, gen)
    return (q * lam) @ q.T


def test_sign_schedule_maps_the_unit_interval_to_one():
    x = torch.cat([torch.logspace(-7, 0, 2001, dtype=torch.float64), torch.linspace(0.9, 1.0005, 200, dtype=torch.float64)])
    for a, b, c in SIGN_SCHEDULE:
        x = a * x + b * x**3 + c * x**5
        assert x.max() < 1.0 + 1e-6 and x.min() > 0.0  # never leaves (0, 1]: no blow-up, no sign change
    for a, b, c in SIGN_SCHEDULE[:14]:
        t = torch.linspace(0, 0.5, 501, dtype=torch.float64)
        assert torch.all(a + 3 * b * t**2 + 5 * c * t**4 >= -1e-9)  # increasing until the band [0.5, 1]
    assert (x - 1).abs().max() < 1e-8


@pytest.mark.parametrize("kind", ["power", "uniform", "clustered", "lowrank", "scalar"])
def test_divide_and_conquer_matches_fp64_eigh(kind):
    gen = torch.Generator().manual_seed(3)
    d = 200
    A64 = _matrix(kind, d, gen)
    lams, vecs, info = eigh_divide_and_conquer(TorchBackend(torch.device("cpu")), [A64.float()], leaf=32)
    assert info["failed"] == []
    lam, Q = lams[0].double(), vecs[0].double()
    ref = torch.linalg.eigvalsh(A64)
    scale = float(ref.abs().max())
    assert torch.all(lam[1:] >= lam[:-1])  # ascending
    assert float((lam - ref).abs().max()) <= 2e-6 * scale
    assert float(torch.linalg.norm(Q.T @ Q - torch.eye(d, dtype=torch.float64))) < 2e-4
    assert float(torch.linalg.norm((Q * lam) @ Q.T - A64)) <= 3e-4 * float(torch.linalg.norm(A64))


def test_batch_of_mixed_sizes_and_small_roots():
    gen = torch.Generator().manual_seed(5)
    mats = [_matrix("power", 150, gen), _matrix("uniform", 20, gen), _matrix("lowrank", 97, gen)]
    lams, vecs, info = eigh_divide_and_conquer(TorchBackend(torch.device("cpu")), [m.float() for m in mats], leaf=32)
    assert info["failed"] == []
    for A, lam, Q in zip(mats, lams, vecs):
        ref = torch.linalg.eigvalsh(A)
        assert float((lam.double() - ref).abs().max()) <= 2e-6 * float(ref.abs().max())
        assert Q.shape == A.shape


def test_unconverged_sign_is_retried_then_reported(monkeypatch):
    """A sign iteration that never yields a projector: the root is given up after the retries and
    reported, the other matrix of the batch is still solved."""
    gen = torch.Generator().manual_seed(7)
    mats = [_matrix("uniform", 80, gen).float(), _matrix("power", 80, gen).float()]
    backend = TorchBackend(torch.device("cpu"))
    original = backend.sign_projector
    attempts = []

    def broken(subs):
        original(subs)
        for s in subs:
            if s.root == 0:
                attempts.append(s.attempt)
                s.idem_err = 1.0  # pretend an eigenvalue sits on the split point

    monkeypatch.setattr(backend, "sign_projector", broken)
    lams, vecs, info = eigh_divide_and_conquer(backend, mats, leaf=32)
    assert info["failed"] == [0] and lams[0] is None and vecs[0] is None
    assert attempts[:3] == [0, 1, 2]
    ref = torch.linalg.eigvalsh(mats[1].double())
    assert float((lams[1].double() - ref).abs().max()) <= 2e-6 * float(ref.abs().max())


def _heavy_tailed(d, gen):
    """A handful of dominant eigenvalues, a power-law tail and a numerically null cluster: the
    shape of a Kronecker factor a few hundred steps into training."""
    lam = torch.cat([1.0 / torch.arange(1, d // 3 + 1, dtype=torch.float64) ** 3, torch.full((d - d // 3,), 1e-12, dtype=torch.float64)])
    q = _orth(d, gen)
    return (q * lam) @ q.T, lam


def test_hints_from_a_previous_decomposition_balance_the_splits():
    gen = torch.Generator().manual_seed(11)
    d = 256
    A64, lam_true = _heavy_tailed(d, gen)
    A = A64.float()
    plain = eigh_divide_and_conquer(TorchBackend(torch.device("cpu")), [A], leaf=32)
    # the hint: last refresh's eigenvalues, at another scale and slightly off
    hint = 3.0 * lam_true * (1 + 0.05 * torch.randn(d, dtype=torch.float64, generator=gen))
    hinted = eigh_divide_and_conquer(TorchBackend(torch.device("cpu")), [A], leaf=32, hints=[hint])
    for lams, vecs, info in (plain, hinted):
        assert info["failed"] == []
        ref = torch.linalg.eigvalsh(A64)
        assert float((lams[0].double() - ref).abs().max()) <= 2e-6 * float(ref.abs().max())
        Q = vecs[0].double()
        assert float(torch.linalg.norm((Q * lams[0].double()) @ Q.T - A64)) <= 3e-4 * float(torch.linalg.norm(A64))
    assert hinted[2]["sign_cubes"] < 0.8 * plain[2]["sign_cubes"]  # less work: the null cluster comes off at once


def test_misleading_hint_costs_one_sign_computation_not_the_result():
    gen = torch.Generator().manual_seed(13)
    d = 120
    A64 = _matrix("uniform", d, gen)
    # a hint whose every gap lies far below the actual spectrum after rescaling by the trace
    hint = torch.cat([torch.full((d // 2,), 1.0), torch.full((d - d // 2,), 1e-9)]).double()
    lams, vecs, info = eigh_divide_and_conquer(TorchBackend(torch.device("cpu")), [A64.float()], leaf=32, hints=[hint])
    assert info["failed"] == []
    ref = torch.linalg.eigvalsh(A64)
    assert float((lams[0].double() - ref).abs().max()) <= 2e-6 * float(ref.abs().max())


def test_second_sign_stage_takes_over_when_an_eigenvalue_sits_at_the_split_point():
    """Eigenvalues 5e-7 of the spread away from the mean are not resolved by the first stage of the
    sign iteration (it reaches about 5e-6): the projector fails the idempotency test and the
    second stage finishes it, at the accuracy of the single long schedule."""
    from optimizers_b200.matrix.eigh_dc import SIGN_STAGES

    assert len(SIGN_STAGES) == 2
    n = 200
    gen = torch.Generator().manual_seed(11)
    q, _ = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=gen))
    lam = torch.linspace(0.0, 1.0, n, dtype=torch.float64)
    gap = 5e-7 * torch.linalg.norm(lam - 0.5)
    lam[n // 2 - 1], lam[n // 2] = 0.5 - gap, 0.5 + gap  # a pair astride the first split point; the mean stays 0.5
    A = ((q * lam) @ q.T)
    backend = TorchBackend(torch.device("cpu"), torch.float64)
    lams, vecs, info = eigh_divide_and_conquer(backend, [A])
    assert info["failed"] == []
    assert info["sign_stages"][1] >= 1, info["sign_stages"]
    ref = torch.linalg.eigvalsh(A)
    assert (lams[0] - ref).abs().max().item() < 1e-10
    V = vecs[0]
    assert (V.T @ V - torch.eye(n, dtype=torch.float64)).abs().max().item() < 1e-10
