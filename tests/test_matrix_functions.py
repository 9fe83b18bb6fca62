"""Matrix functions: closed-form expectations and agreement with the reference implementation."""

from fractions import Fraction

import pytest
import torch

from optimizers_b200.config import (
    CoupledHigherOrderConfig,
    CoupledNewtonConfig,
    EigenConfig,
    EighEigendecompositionConfig,
    NewtonSchulzOrthogonalizationConfig,
    PerturbationConfig,
    PseudoInverseConfig,
    QREigendecompositionConfig,
    SVDOrthogonalizationConfig,
)
from optimizers_b200.matrix import functions as mf

ROOT_CONFIGS = [
    EigenConfig(),
    EigenConfig(rank_deficient_stability_config=PerturbationConfig(perturb_before_computation=False)),
    CoupledNewtonConfig(),
    CoupledHigherOrderConfig(rel_epsilon=0.0, abs_epsilon=0.0),
    CoupledHigherOrderConfig(rel_epsilon=0.0, abs_epsilon=0.0, order=2),
    CoupledHigherOrderConfig(rel_epsilon=0.0, abs_epsilon=0.0, order=5),
]


@pytest.mark.parametrize("cfg", ROOT_CONFIGS, ids=lambda c: type(c).__name__ + str(getattr(c, "order", "")))
def test_inverse_root_known_matrices(cfg):
    A = torch.tensor([[1.0, 0.0], [0.0, 4.0]])
    X = mf.matrix_inverse_root(A, Fraction(2), cfg)
    torch.testing.assert_close(X, torch.tensor([[1.0, 0.0], [0.0, 0.5]]), atol=0.05, rtol=1e-2)
    B = torch.tensor([[1195.0, -944.0, -224.0], [-944.0, 746.0, 177.0], [-224.0, 177.0, 42.0]])
    Y = mf.matrix_inverse_root(B, Fraction(2), cfg)
    want = torch.tensor([[1.0, 1.0, 1.0], [1.0, 2.0, 1.0], [1.0, 1.0, 7.0]])  # B = inverse(want)^2 up to rounding
    torch.testing.assert_close(Y @ Y @ B, torch.eye(3), atol=0.2, rtol=0.2)
    assert want.shape == Y.shape


@pytest.mark.parametrize("root", [2, 4, 8])
@pytest.mark.parametrize("n", [10, 100])
def test_coupled_newton_on_tridiagonal_family(root, n):
    torch.manual_seed(0)
    A = 2 * torch.eye(n) + torch.diag(torch.full((n - 1,), -0.5), 1) + torch.diag(torch.full((n - 1,), -0.5), -1)
    X, M, flag, iters, err = mf._inverse_root_coupled_newton(A, root, 0.0, 100, 1e-6)
    assert flag == mf.NewtonConvergenceFlag.CONVERGED and err <= 1e-6
    lam, Q = torch.linalg.eigh(A.double())
    want = (Q * lam.pow(-1.0 / root)) @ Q.T
    torch.testing.assert_close(X.double(), want, atol=1e-4, rtol=1e-4)


def test_inverse_root_argument_checks():
    with pytest.raises(ValueError, match="not 2-dimensional"):
        mf.matrix_inverse_root(torch.zeros(2, 2, 2), Fraction(2))
    with pytest.raises(ValueError, match="not square"):
        mf.matrix_inverse_root(torch.zeros(2, 3), Fraction(2))
    with pytest.raises(ValueError, match="should be positive"):
        mf.matrix_inverse_root(torch.eye(2), Fraction(-1))
    with pytest.raises(ValueError, match="must be equal to 1"):
        mf.matrix_inverse_root(torch.eye(2), Fraction(3, 2), CoupledNewtonConfig())
    with pytest.raises(ValueError, match="should be 0.0 when using pseudo-inverse"):
        mf.matrix_inverse_root(
            torch.eye(2), Fraction(2), EigenConfig(rank_deficient_stability_config=PseudoInverseConfig()), epsilon=1e-3
        )


def test_pseudo_inverse_drops_null_space():
    A = torch.diag(torch.tensor([4.0, 0.0, 1.0]))
    X = mf.matrix_inverse_root(A, Fraction(2), EigenConfig(rank_deficient_stability_config=PseudoInverseConfig()))
    torch.testing.assert_close(X, torch.diag(torch.tensor([0.5, 0.0, 1.0])))


def test_negative_eigenvalues_are_shifted_to_epsilon():
    L = torch.tensor([-0.5, 1.0, 2.0])
    s = mf.stabilized_inverse_power(L, 2, 0.1, PerturbationConfig(perturb_before_computation=True))
    torch.testing.assert_close(s, (L + 0.5 + 0.1).pow(-0.5))
    s = mf.stabilized_inverse_power(torch.tensor([0.5, 1.0]), 2, 0.1, PerturbationConfig(perturb_before_computation=True))
    torch.testing.assert_close(s, torch.tensor([0.5, 1.0]).pow(-0.5))  # already above epsilon: untouched
    s = mf.stabilized_inverse_power(torch.tensor([0.5, 1.0]), 2, 0.1, PerturbationConfig(perturb_before_computation=False))
    torch.testing.assert_close(s, torch.tensor([0.6, 1.1]).pow(-0.5))


def test_eigendecomposition_eigh_qr_and_tolerance():
    torch.manual_seed(1)
    Q0, _ = torch.linalg.qr(torch.randn(6, 6))
    lam0 = torch.tensor([0.1, 0.5, 1.0, 2.0, 3.0, 10.0])
    A = (Q0 * lam0) @ Q0.T
    lam, Q = mf.matrix_eigendecomposition(A)
    torch.testing.assert_close(lam, lam0, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close((Q * lam) @ Q.T, A, atol=1e-4, rtol=1e-4)
    # QR iteration from the exact basis stays there; from identity with many iterations it converges
    lam_q, V = mf.matrix_eigendecomposition(A, eigendecomposition_config=QREigendecompositionConfig(), eigenvectors_estimate=Q)
    torch.testing.assert_close(lam_q, lam0, atol=1e-4, rtol=1e-4)
    lam_q, V = mf.matrix_eigendecomposition(
        A, eigendecomposition_config=QREigendecompositionConfig(max_iterations=500, tolerance=1e-6), eigenvectors_estimate=torch.eye(6)
    )
    torch.testing.assert_close(lam_q, lam0, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(V.T @ V, torch.eye(6), atol=1e-4, rtol=1e-4)
    # tolerance: a basis that already diagonalises A is returned as is
    cfg = EighEigendecompositionConfig(tolerance=0.01)
    lam_t, Q_t = mf.matrix_eigendecomposition(A, eigendecomposition_config=cfg, eigenvectors_estimate=Q)
    assert Q_t is Q
    with pytest.raises(ValueError, match="eigenvectors_estimate should be passed"):
        mf.matrix_eigendecomposition(A, eigendecomposition_config=cfg)


def test_orthogonalization():
    torch.manual_seed(2)
    for shape in [(8, 5), (5, 8), (6, 6)]:
        A = torch.randn(*shape)
        U = mf.matrix_orthogonalization(A, SVDOrthogonalizationConfig())
        k = min(shape)
        gram = U.T @ U if shape[0] >= shape[1] else U @ U.T
        torch.testing.assert_close(gram, torch.eye(k), atol=1e-4, rtol=1e-4)
        N = mf.matrix_orthogonalization(A, NewtonSchulzOrthogonalizationConfig(num_iterations=12))
        s = torch.linalg.svdvals(N)
        assert s.max() < 1.3 and s.min() > 0.5  # quintic Newton-Schulz keeps singular values in a band near 1
    scaled = mf.matrix_orthogonalization(
        torch.eye(3), SVDOrthogonalizationConfig(scale_by_dims_fn=lambda d_in, d_out: 2.0, scale_by_nuclear_norm=True)
    )
    torch.testing.assert_close(scaled, 6.0 * torch.eye(3))


def test_against_reference_matrix_functions():
    from ref_oracle import reference, reference_available

    if not reference_available():
        pytest.skip("reference not installed")
    R = reference()
    from distributed_shampoo.preconditioner import matrix_functions as rmf

    torch.manual_seed(3)
    for n in (3, 17, 64):
        G = torch.randn(n, 2 * n)
        A = G @ G.T / n
        pairs = [
            (EigenConfig(), R.EigenConfig()),
            (CoupledNewtonConfig(), R.CoupledNewtonConfig()),
            (CoupledHigherOrderConfig(rel_epsilon=1e-8, abs_epsilon=1e-12), R.CoupledHigherOrderConfig(rel_epsilon=1e-8, abs_epsilon=1e-12)),
        ]
        for ours, theirs in pairs:
            for root in (2, 4):
                a = mf.matrix_inverse_root(A, Fraction(root), ours, epsilon=1e-6)
                b = rmf.matrix_inverse_root(A, Fraction(root), theirs, epsilon=1e-6)
                assert torch.equal(a, b), (type(ours).__name__, n, root, (a - b).abs().max())
        Q0 = torch.linalg.qr(torch.randn(n, n))[0]
        a = mf.matrix_eigendecomposition(A, 1e-6, QREigendecompositionConfig(max_iterations=3), Q0)
        b = rmf.matrix_eigendecomposition(A, 1e-6, R.QREigendecompositionConfig(max_iterations=3), Q0)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
        X = torch.randn(n, n + 5)
        assert torch.equal(mf.matrix_orthogonalization(X), rmf.matrix_orthogonalization(X))


def _reference_pair():
    from ref_oracle import reference, reference_available

    if not reference_available():
        pytest.skip("reference not installed")
    R = reference()
    from distributed_shampoo.preconditioner import matrix_functions as rmf

    return R, rmf


def _same(call_ours, call_theirs, label):
    """Both return equal tensors (bit for bit), or both raise the same kind of error."""
    try:
        want = call_theirs()
    except Exception as error:  # noqa: BLE001
        with pytest.raises(type(error).__mro__[0] if type(error).__module__ == "builtins" else Exception):
            call_ours()
        return
    got = call_ours()
    want, got = (want if isinstance(want, tuple) else (want,)), (got if isinstance(got, tuple) else (got,))
    assert len(want) == len(got), label
    for a, b in zip(want, got):
        assert a.shape == b.shape and a.dtype == b.dtype and torch.equal(a, b), (label, (a.double() - b.double()).abs().max().item())


def _test_matrices():
    gen = torch.Generator().manual_seed(9)
    out = {}
    G = torch.randn(12, 30, generator=gen)
    out["full_rank"] = G @ G.T / 30
    L = torch.randn(12, 3, generator=gen)
    out["rank_3_of_12"] = L @ L.T
    out["diagonal"] = torch.diag(torch.linspace(0.1, 3.0, 7))
    out["one_by_one"] = torch.tensor([[2.5]])
    out["tiny_scale"] = out["full_rank"] * 1e-20
    out["with_negative_eigenvalue"] = out["full_rank"] - 0.5 * torch.eye(12)
    out["float64"] = out["full_rank"].double()
    return out


def test_inverse_roots_against_reference_on_a_grid_of_configurations():
    R, rmf = _reference_pair()
    stabilities = [
        (lambda L: L.PerturbationConfig(), "perturb_before"),
        (lambda L: L.PerturbationConfig(perturb_before_computation=False), "perturb_after"),
        (lambda L: L.PseudoInverseConfig(), "pseudo_inverse"),
        (lambda L: L.PseudoInverseConfig(rank_atol=1e-6, rank_rtol=1e-4), "pseudo_inverse_tolerances"),
    ]
    import optimizers_b200.config as ours_lib
    import distributed_shampoo.preconditioner.matrix_functions_types as theirs_lib

    for name, A in _test_matrices().items():
        for make_stability, stability_name in stabilities:
            for retry in (True, False):
                for root in (Fraction(2), Fraction(4), Fraction(3, 2), Fraction(1)):
                    for epsilon in (0.0, 1e-6):
                        ours = ours_lib.EigenConfig(rank_deficient_stability_config=make_stability(ours_lib), retry_double_precision=retry)
                        theirs = theirs_lib.EigenConfig(rank_deficient_stability_config=make_stability(theirs_lib), retry_double_precision=retry)
                        _same(
                            lambda: mf.matrix_inverse_root(A, root, ours, epsilon=epsilon),
                            lambda: rmf.matrix_inverse_root(A, root, theirs, epsilon=epsilon),
                            (name, stability_name, retry, root, epsilon),
                        )
        for root in (Fraction(2), Fraction(4), Fraction(3, 2)):
            for iterations, tolerance in ((100, 1e-6), (3, 1e-12)):
                _same(
                    lambda: mf.matrix_inverse_root(A, root, ours_lib.CoupledNewtonConfig(max_iterations=iterations, tolerance=tolerance), epsilon=1e-6),
                    lambda: rmf.matrix_inverse_root(A, root, theirs_lib.CoupledNewtonConfig(max_iterations=iterations, tolerance=tolerance), epsilon=1e-6),
                    (name, "newton", root, iterations),
                )
            for order in (2, 3, 4, 6):
                kw = dict(rel_epsilon=1e-8, abs_epsilon=1e-12, order=order, max_iterations=40, tolerance=1e-8)
                _same(
                    lambda: mf.matrix_inverse_root(A, root, ours_lib.CoupledHigherOrderConfig(**kw)),
                    lambda: rmf.matrix_inverse_root(A, root, theirs_lib.CoupledHigherOrderConfig(**kw)),
                    (name, "higher_order", root, order),
                )


def test_eigendecompositions_and_orthogonalizations_against_reference_on_a_grid():
    R, rmf = _reference_pair()
    import optimizers_b200.config as ours_lib
    import distributed_shampoo.preconditioner.matrix_functions_types as theirs_lib

    gen = torch.Generator().manual_seed(4)
    for name, A in _test_matrices().items():
        n = A.shape[0]
        estimate = torch.linalg.qr(torch.randn(n, n, generator=gen, dtype=A.dtype))[0]
        for epsilon in (0.0, 1e-6):
            for tolerance in (0.0, 1e-2):
                for make, label in (
                    (lambda L: L.EighEigendecompositionConfig(tolerance=tolerance), "eigh"),
                    (lambda L: L.EighEigendecompositionConfig(tolerance=tolerance, retry_double_precision=False), "eigh_no_retry"),
                    (lambda L: L.QREigendecompositionConfig(max_iterations=1, tolerance=tolerance), "qr_1"),
                    (lambda L: L.QREigendecompositionConfig(max_iterations=5, tolerance=tolerance), "qr_5"),
                ):
                    for guess in (estimate, torch.eye(n, dtype=A.dtype)):
                        _same(
                            lambda: mf.matrix_eigendecomposition(A, epsilon, make(ours_lib), guess),
                            lambda: rmf.matrix_eigendecomposition(A, epsilon, make(theirs_lib), guess),
                            (name, label, epsilon, tolerance),
                        )
    for shape in ((5, 5), (4, 9), (9, 4), (1, 6)):
        X = torch.randn(*shape, generator=gen)
        for make, label in (
            (lambda L: L.SVDOrthogonalizationConfig(), "svd"),
            (lambda L: L.SVDOrthogonalizationConfig(scale_by_nuclear_norm=True), "svd_nuclear"),
            (lambda L: L.NewtonSchulzOrthogonalizationConfig(), "newton_schulz"),
            (lambda L: L.NewtonSchulzOrthogonalizationConfig(num_iterations=2, coefficients=(1.5, -0.5, 0.0)), "newton_schulz_cubic"),
        ):
            _same(lambda: mf.matrix_orthogonalization(X, make(ours_lib)), lambda: rmf.matrix_orthogonalization(X, make(theirs_lib)), (shape, label))
