"""Host logic of the batched coupled iterations (optimizers_b200/matrix/batched.py) on the CPU.

The launch tables, the ping-pong of the iterates, the Horner construction of the higher-order map,
the stopping rules, the final verification and the power of a fractional root are plain Python
around the extension's calls.  Here the extension is replaced by a stand-in that performs every
call with torch on the CPU, and the results are compared with the per-factor torch functions
(``matrix/functions.py``, themselves pinned against the reference's).
"""

from fractions import Fraction
from types import SimpleNamespace

import pytest
import torch

from optimizers_b200 import (
    CoupledHigherOrderConfig,
    CoupledNewtonConfig,
    DistributedShampoo,
    RootInvShampooPreconditionerConfig,
)
from fake_ext import FakeExt
from optimizers_b200.matrix import batched, functions as mf


def _blocks(config, exponent=None, seed=0):
    torch.manual_seed(seed)
    model = torch.nn.Sequential(torch.nn.Linear(20, 24), torch.nn.Tanh(), torch.nn.Linear(24, 6))
    override = {} if exponent is None else {2: exponent}
    opt = DistributedShampoo(
        model.parameters(), lr=1e-3, epsilon=1e-6, max_preconditioner_dim=16, precondition_frequency=100,
        start_preconditioning_step=100,
        preconditioner_config=RootInvShampooPreconditionerConfig(
            amortized_computation_config=config, inverse_exponent_override=override
        ),
    )
    for _ in range(3):
        opt.zero_grad()
        model(torch.randn(64, 20)).square().mean().backward()
        opt.step()
    plist = opt._per_group_state_lists[0]["shampoo_preconditioner_list"]
    return [SimpleNamespace(factors=kf, inv_hi=[torch.zeros(1)]) for kf in plist._local_kronecker_factors_unwrapped]


def _residual(A_r, X, root):
    """max |A_r X^p - I| with X^p recovered from the returned X^q of a root p / q, in fp64."""
    lam, Q = torch.linalg.eigh(X.double())
    Xp = (Q * lam.clamp(min=0).pow(root.numerator / root.denominator)) @ Q.T
    return (A_r.double() @ Xp - torch.eye(A_r.shape[0], dtype=torch.float64)).abs().max().item()


def _check(blocks, config, slack):
    """These factors are ill-conditioned (ridge 1e-6 of the norm), so the per-factor function and
    the batched loop both return roots with a visible residual: the loop's must not be worse than
    ``slack`` times the function's (plus a floor)."""
    checked = 0
    for b in blocks:
        kf = b.factors
        for F, X, root in zip(kf.get_unpacked_factor_matrices(), kf.get_unpacked_inv_factor_matrices(), kf.roots):
            root = Fraction(root)
            want = mf.matrix_inverse_root(F, root, config, epsilon=kf.epsilon)
            if isinstance(config, CoupledNewtonConfig):
                ridge = kf.epsilon
            else:
                ridge = max(F.abs().sum(dim=1).max().item() * config.rel_epsilon, config.abs_epsilon)
            A_r = F + ridge * torch.eye(F.shape[0])
            mine, ref = _residual(A_r, X, root), _residual(A_r, want, root)
            assert mine <= slack * ref + 1e-3, (F.shape, root, mine, ref)
            scale = want.abs().max().item()
            assert (X - want).abs().max().item() <= 20 * max(mine, ref, 1e-4) * scale, (F.shape, root)
            checked += 1
    assert checked >= 6


def test_coupled_newton_loop_matches_the_per_factor_function():
    config = CoupledNewtonConfig(max_iterations=100, tolerance=1e-6)
    blocks = _blocks(config)
    batched.batched_newton_refresh(FakeExt(), blocks, 1.0, True, torch.zeros(1, dtype=torch.int32))
    _check(blocks, config, 3.0)


@pytest.mark.parametrize("order,exponent", [(2, None), (3, None), (4, 0.5), (3, 2.0 / 3.0), (5, 1.0)])
def test_higher_order_loop_matches_the_per_factor_function(order, exponent):
    config = CoupledHigherOrderConfig(rel_epsilon=1e-6, abs_epsilon=1e-10, order=order, tolerance=1e-6, max_iterations=100)
    blocks = _blocks(config, exponent)
    ext = FakeExt()
    batched.batched_newton_refresh(ext, blocks, 1.0, True, torch.zeros(1, dtype=torch.int32))
    assert ext.gemm_launches > 0
    _check(blocks, config, 3.0)


def test_higher_order_verification_rejects_a_wrong_root():
    """A factor whose iteration is cut off after two steps fails the A_r X^p check and keeps its
    previous inverse root; the others are unaffected."""
    config = CoupledHigherOrderConfig(rel_epsilon=1e-12, abs_epsilon=1e-12, order=3, tolerance=1e-6, max_iterations=2)
    blocks = _blocks(config)
    before = [[m.clone() for m in b.factors.inv_factor_matrices] for b in blocks]
    batched.batched_newton_refresh(FakeExt(), blocks, 1.0, True, torch.zeros(1, dtype=torch.int32))
    kept = sum(
        torch.equal(m, old) for b, olds in zip(blocks, before) for m, old in zip(b.factors.inv_factor_matrices, olds)
    )
    assert kept >= 1


@pytest.mark.parametrize("max_iterations", [1, 3])
def test_qr_iteration_loop_matches_the_per_factor_function(max_iterations):
    """The batched warm-started QR iteration against the per-factor torch function: same number of
    sweeps (the criterion is evaluated the same way), hence the same bases up to column signs."""
    gen = torch.Generator().manual_seed(5)
    mats, estimates = [], []
    for n in (12, 40, 7):
        q, _ = torch.linalg.qr(torch.randn(n, n, generator=gen))
        lam = torch.linspace(1.0, 3.0, n)
        mats.append((q * lam) @ q.T)
        # previous eigenvectors: the true ones rotated a little
        skew = torch.randn(n, n, generator=gen) * 0.03
        estimates.append(q @ torch.linalg.matrix_exp(skew - skew.T))
    estimates[2] = torch.linalg.eigh(mats[2])[1]  # already diagonalising: must be left alone
    status = torch.zeros(1, dtype=torch.int32)
    got = batched.native_qr_iteration(FakeExt(), mats, estimates, max_iterations, 1e-4, status)
    for A, V0, V in zip(mats, estimates, got):
        _, want = mf._qr_iteration(A, V0, max_iterations, 1e-4)
        n = A.shape[0]
        assert torch.allclose(V.T @ V, torch.eye(n), atol=1e-5)
        overlap = (want.T @ V).abs()
        assert torch.allclose(overlap, torch.eye(n), atol=2e-3), overlap
    assert torch.allclose(got[2].abs(), estimates[2].abs(), atol=1e-6)


@pytest.mark.parametrize("split", [True, False])
def test_newton_schulz_loop_matches_the_per_factor_function(split):
    gen = torch.Generator().manual_seed(6)
    shapes = [(20, 12), (9, 30), (16, 16)]
    mats = [torch.randn(*s, generator=gen) for s in shapes]
    coefficients = (3.4445, -4.7750, 2.0315)
    runner = batched.BatchedNewtonSchulz(FakeExt(), shapes, torch.device("cpu"), split=split)
    got = runner(mats, 5, coefficients)
    for A, X in zip(mats, got):
        want = mf.newton_schulz(A, 5, coefficients)
        assert X.shape == A.shape
        assert torch.allclose(X, want, rtol=1e-4, atol=1e-4)
