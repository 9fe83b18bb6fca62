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
from optimizers_b200.matrix import batched, functions as mf


class FakeExt:
    """The subset of the extension's interface that the coupled iterations use."""

    FLAG_PACKED_C, FLAG_SPLIT_OUT, FLAG_SUMSQ, FLAG_NO_C = 1, 2, 4, 8
    FLAG_MIRROR, FLAG_ADD_DIAG = 64, 128

    def __init__(self):
        self.gemm_launches = 0

    def tf32_split(self, src, hi, lo):
        hi.copy_(src)
        lo.zero_()

    def build_mat_table(self, specs):
        return (list(specs), None, 0)

    def affine_identity_split(self, specs, _chunks, _n, a, b):
        for src, hi, lo, _err in specs:
            hi.copy_(a * src + b * torch.eye(src.shape[0]))
            if lo is not None:
                lo.zero_()

    def identity_error(self, specs, _chunks, _n):
        for src, _hi, _lo, err in specs:
            err[0] = (src - torch.eye(src.shape[0])).abs().max()

    def build_gemm_plan(self, specs):
        return (list(specs), None, 0)

    def run_gemm_plan(self, specs, _tiles, _n, alpha, beta, split, status, gamma=0.0):
        self.gemm_launches += 1
        for a_hi, a_lo, b_hi, b_lo, c, d_hi, d_lo, _sumsq, _ldc, _ldd, flags, _upper in specs:
            A = a_hi + (a_lo if a_lo is not None else 0)
            B = b_hi + (b_lo if b_lo is not None else 0)
            out = alpha * (A.double() @ B.double().T).float()
            m, n = out.shape  # outputs may be handed over in their padded storage
            if flags & self.FLAG_MIRROR:
                assert _upper and m == n
                out = torch.triu(out) + torch.triu(out, 1).T
            if c is not None and not flags & self.FLAG_NO_C and beta != 0.0:
                out = out + beta * c[:m, :n]
            if flags & self.FLAG_ADD_DIAG:
                out = out + gamma * torch.eye(m)
            if c is not None and not flags & self.FLAG_NO_C:
                c[:m, :n].copy_(out)
            if flags & self.FLAG_SPLIT_OUT:
                d_hi[:m, :n].copy_(out)
                d_lo.zero_()


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
