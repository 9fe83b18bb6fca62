"""Matrix functions behind the amortised preconditioner refresh: inverse p-th roots,
symmetric eigendecompositions and semi-orthogonalisation.

This module is the device-agnostic implementation written with torch operators; it is what runs
on CPU, it is the numerical oracle for the sm_100a kernels in ``optimizers_b200.ops``, and it is
the fallback for shapes the kernels reject.  ``matrix_inverse_root``,
``matrix_eigendecomposition`` and ``matrix_orthogonalization`` route to the native batched
kernels through ``optimizers_b200.ops`` when the operand lives on a B200 and the native back-end
is enabled (see ``optimizers_b200.matrix.batched``).

Behaviour follows the reference's ``distributed_shampoo/preconditioner/matrix_functions.py``:
inverse root from an eigendecomposition (:179-279), eigen / coupled Newton / coupled higher-order
root inverse (:283-693), eigh with fp64 retry and offload, tolerance criterion and QR iteration
(:699-908), SVD and Newton-Schulz orthogonalisation (:912-1022).
"""

from __future__ import annotations

import enum
import logging
import math
from fractions import Fraction

import torch
from torch import Tensor

from optimizers_b200.config import (
    CoupledHigherOrderConfig,
    CoupledNewtonConfig,
    DefaultEigenConfig,
    DefaultEigendecompositionConfig,
    DefaultNewtonSchulzOrthogonalizationConfig,
    DefaultPerturbationConfig,
    EigenConfig,
    EigendecompositionConfig,
    EighEigendecompositionConfig,
    NewtonSchulzOrthogonalizationConfig,
    OrthogonalizationConfig,
    PerturbationConfig,
    PseudoInverseConfig,
    QREigendecompositionConfig,
    RankDeficientStabilityConfig,
    RootInvConfig,
    SVDOrthogonalizationConfig,
)

logger: logging.Logger = logging.getLogger(__name__)


class NewtonConvergenceFlag(enum.Enum):
    REACHED_MAX_ITERS = 0
    CONVERGED = 1
    EARLY_STOP = 2


def _require_2d(A: Tensor) -> None:
    if A.dim() != 2:
        raise ValueError(f"Matrix is not 2-dimensional! A.shape={A.shape}")


def _require_square(A: Tensor) -> None:
    _require_2d(A)
    if A.shape[0] != A.shape[1]:
        raise ValueError(f"Matrix is not square! A.shape={A.shape}")


def _ridge(A: Tensor, epsilon: float | Tensor) -> Tensor:
    """A + εI (returns A itself when ε is the number 0)."""
    if isinstance(epsilon, (int, float)) and epsilon == 0:
        return A
    out = A.clone()
    out.diagonal().add_(epsilon)
    return out


# --------------------------------------------------------------------------------------------
# Inverse root from (λ, Q)
# --------------------------------------------------------------------------------------------
def stabilized_inverse_power(
    L: Tensor,
    root: Fraction | float,
    epsilon: float,
    rank_deficient_stability_config: RankDeficientStabilityConfig,
    lambda_min: Tensor | float | None = None,
) -> Tensor:
    """λ ↦ λ^(-1/root) after the configured treatment of small or negative eigenvalues.  Runs
    without a host synchronisation (the comparison with ε is a ``torch.where``)."""
    inv = -1.0 / float(root)
    match rank_deficient_stability_config:
        case PseudoInverseConfig(rank_atol=atol, rank_rtol=rtol):
            if epsilon != 0.0:
                raise ValueError(f"{epsilon=} should be 0.0 when using pseudo-inverse!")
            if rtol is None:
                rtol = L.numel() * torch.finfo(L.dtype).eps
            cutoff = torch.clamp(rtol * L.max().relu(), min=atol)
            return torch.where(L <= cutoff, torch.zeros_like(L), L.pow(inv))
        case PerturbationConfig(perturb_before_computation=before):
            lo = L.min() if lambda_min is None else lambda_min
            lo = torch.as_tensor(lo, dtype=L.dtype, device=L.device)
            if before:
                # ε was already added to the matrix; only repair what is still below ε.
                fixed = torch.where(lo < epsilon, (L - lo) + epsilon, L)
            else:
                fixed = (L - torch.clamp(lo, max=0.0)) + epsilon
            return fixed.pow(inv)
        case _:
            raise NotImplementedError(f"{rank_deficient_stability_config=} is not supported.")


def matrix_inverse_root_from_eigendecomposition(
    L: Tensor,
    Q: Tensor,
    root: Fraction,
    epsilon: float = 0.0,
    rank_deficient_stability_config: RankDeficientStabilityConfig = DefaultPerturbationConfig,
) -> Tensor:
    """Q · diag(λ^(-1/root)) · Qᵀ."""
    scaled = stabilized_inverse_power(L, root, epsilon, rank_deficient_stability_config)
    return (Q * scaled.unsqueeze(0)) @ Q.T


# --------------------------------------------------------------------------------------------
# Inverse root algorithms
# --------------------------------------------------------------------------------------------
def _inverse_root_eigen(A: Tensor, root: Fraction, epsilon: float, cfg: EigenConfig):
    if root <= 0:
        raise ValueError(f"Root {root} should be positive!")
    L, Q = matrix_eigendecomposition(
        A,
        epsilon=epsilon,
        eigendecomposition_config=EighEigendecompositionConfig(
            rank_deficient_stability_config=cfg.rank_deficient_stability_config,
            retry_double_precision=cfg.retry_double_precision,
            eigendecomposition_offload_device=cfg.eigendecomposition_offload_device,
            tolerance=0.0,
        ),
    )
    X = matrix_inverse_root_from_eigendecomposition(
        L, Q, root, epsilon, cfg.rank_deficient_stability_config
    )
    return X, L, Q


def _inverse_root_coupled_newton(
    A: Tensor, root: int, epsilon: float, max_iterations: int, tolerance: float
):
    """Coupled Newton iteration X_{k+1} = X_k M_p, M_{k+1} = M_p^p M_k with
    M_p = (1-α) I + α M_k, α = -1/p; starts from z = (p+1)/(2‖A‖_F)."""
    n = A.shape[0]
    alpha = -1.0 / root
    eye = torch.eye(n, dtype=A.dtype, device=A.device)
    A_r = _ridge(A, epsilon)
    z = (root + 1) / (2 * torch.linalg.norm(A_r))
    X = z ** (-alpha) * eye
    M = z * A_r
    err = torch.dist(M, eye, p=torch.inf)
    it = 0
    while err > tolerance and it < max_iterations:
        it += 1
        M_p = M.mul(alpha).add_(eye, alpha=1 - alpha)
        X = X @ M_p
        M = torch.linalg.matrix_power(M_p, root) @ M
        err = torch.dist(M, eye, p=torch.inf)
    flag = NewtonConvergenceFlag.CONVERGED if err <= tolerance else NewtonConvergenceFlag.REACHED_MAX_ITERS
    return X, M, flag, it, err


def _inverse_root_higher_order(A: Tensor, root: Fraction, cfg: CoupledHigherOrderConfig):
    """Coupled iteration of order ``cfg.order`` for A^(-q/p): Taylor coefficients of
    (1-x)^(-1/p) evaluated by Horner in the residual I - M; one Newton step first; stops early
    when the residual grows by 20 % or stalls; verifies ‖A X^p - I‖∞ ≤ 0.1 at the end."""
    saved_tf32 = torch.backends.cuda.matmul.allow_tf32
    if cfg.disable_tf32:
        torch.backends.cuda.matmul.allow_tf32 = False
    try:
        p, q = root.numerator, root.denominator
        if min(abs(p), abs(q)) >= 10:
            logger.warning(
                f"abs(root.numerator)={abs(p)} and abs(root.denominator)={abs(q)} are probably too big for best performance."
            )
        order = cfg.order
        coeff = [1.0]
        num = den = 1
        for i in range(1, order):
            num *= 1 + (i - 1) * p
            den *= i * p
            coeff.append(num / den)

        n = A.shape[0]
        s = -1.0 / p
        lam = torch.linalg.matrix_norm(A, torch.inf)
        if not math.isfinite(lam):
            raise ArithmeticError("Input matrix has entries close to inf, exiting root inverse")
        eps = torch.clamp(lam * cfg.rel_epsilon, min=cfg.abs_epsilon)
        eye = torch.eye(n, dtype=A.dtype, device=A.device)
        A_r = _ridge(A, eps)
        z = torch.reciprocal(torch.trace(A_r))
        X = torch.pow(z, -s) * eye
        M = z * A_r

        def residual(M: Tensor) -> Tensor:
            return torch.linalg.vector_norm(M - eye, torch.inf)

        # One plain Newton step to enter the convergence region of the higher-order map.
        M_p = M.mul(s).add_(eye, alpha=1 - s)
        X = X @ M_p
        M = torch.linalg.matrix_power(M_p, p) @ M
        err = residual(M)
        it = 1
        flag = None
        while err > cfg.tolerance and it < cfg.max_iterations:
            it += 1
            R = eye - M
            M_p = R.mul(coeff[order - 1]).add_(eye, alpha=coeff[order - 2])
            for i in reversed(range(order - 2)):
                M_p = torch.addmm(eye, M_p, R, beta=coeff[i])
            X = X @ M_p
            M = torch.linalg.matrix_power(M_p, p) @ M
            new_err = residual(M)
            if new_err > err * 1.2 or (new_err == err and err < 1e-3):
                flag = NewtonConvergenceFlag.EARLY_STOP
                break
            err = new_err
        if flag is None:
            flag = (
                NewtonConvergenceFlag.REACHED_MAX_ITERS
                if err > cfg.tolerance
                else NewtonConvergenceFlag.CONVERGED
            )
        true_err = torch.linalg.vector_norm(A_r @ torch.linalg.matrix_power(X, p) - eye, torch.inf)
        if true_err > 1e-1:
            raise ArithmeticError(
                f"Error in matrix inverse root (before powering for fractions) {true_err} exceeds threshold 1e-1, raising an exception!"
            )
        if q > 1:
            X = torch.linalg.matrix_power(X, q)
        if not torch.isfinite(X).all():
            raise ArithmeticError(
                "NaN/Inf in matrix inverse root (after powering for fractions), raising an exception!"
            )
        return X, M, flag, it, true_err
    finally:
        torch.backends.cuda.matmul.allow_tf32 = saved_tf32


def matrix_inverse_root(
    A: Tensor,
    root: Fraction,
    root_inv_config: RootInvConfig = DefaultEigenConfig,
    epsilon: float = 0.0,
) -> Tensor:
    """(A + εI)^(-1/root) of a symmetric positive semi-definite matrix."""
    _require_square(A)
    match root_inv_config:
        case EigenConfig():
            X, _, _ = _inverse_root_eigen(A, root, epsilon, root_inv_config)
        case CoupledNewtonConfig(max_iterations=iters, tolerance=tol):
            if root.denominator != 1:
                raise ValueError(
                    f"root.denominator={root.denominator} must be equal to 1 to use coupled inverse Newton iteration!"
                )
            X, _, flag, _, _ = _inverse_root_coupled_newton(A, root.numerator, epsilon, iters, tol)
            if flag == NewtonConvergenceFlag.REACHED_MAX_ITERS:
                logger.warning("Newton did not converge and reached maximum number of iterations!")
        case CoupledHigherOrderConfig():
            X, _, flag, _, _ = _inverse_root_higher_order(A, root, root_inv_config)
            if flag == NewtonConvergenceFlag.REACHED_MAX_ITERS:
                logger.warning(
                    "Higher order method did not converge and reached maximum number of iterations!"
                )
        case _:
            raise NotImplementedError(
                f"Root inverse config is not implemented! Specified root inverse config is root_inv_config={root_inv_config}."
            )
    return X


# --------------------------------------------------------------------------------------------
# Eigendecomposition
# --------------------------------------------------------------------------------------------
def _eigh(A: Tensor, retry_double_precision: bool, offload_device: str) -> tuple[Tensor, Tensor]:
    home_device, home_dtype = A.device, A.dtype
    if offload_device != "":
        A = A.to(device=offload_device)
    try:
        L, Q = torch.linalg.eigh(A)
    except Exception as exception:
        if not (retry_double_precision and A.dtype != torch.float64):
            raise exception
        logger.warning(
            f"Failed to compute eigendecomposition in {A.dtype} precision with exception {exception}! Retrying in double precision..."
        )
        L, Q = torch.linalg.eigh(A.double())
    return L.to(device=home_device, dtype=home_dtype), Q.to(device=home_device, dtype=home_dtype)


def _nearly_diagonal(B: Tensor, tolerance: float) -> bool:
    """‖B - diag B‖_F ≤ tolerance·‖B‖_F."""
    total = torch.linalg.norm(B)
    diag = torch.linalg.norm(B.diag())
    off = torch.sqrt(total**2 - diag**2)
    return bool(off <= tolerance * total)


def _qr_iteration(
    A: Tensor, eigenvectors_estimate: Tensor, max_iterations: int, tolerance: float
) -> tuple[Tensor, Tensor]:
    """Warm-started orthogonal iteration in the basis of the previous eigenvectors: B = QᵀAQ,
    then repeatedly B = RQ' with Q'R = B, accumulating Q ← QQ'.  Eigenvalue estimates are the
    diagonal of B, returned ascending with the columns permuted to match."""
    V = eigenvectors_estimate
    assert V.dtype == A.dtype, f"V.dtype={V.dtype} does not match A.dtype={A.dtype}!"
    B = V.T @ A @ V
    it = 0
    while it < max_iterations and not _nearly_diagonal(B, tolerance):
        Qs, Rs = torch.linalg.qr(B)
        B = Rs @ Qs
        V = V @ Qs
        it += 1
    lam, order = B.diag().sort(stable=True)
    return lam, V[:, order]


def matrix_eigendecomposition(
    A: Tensor,
    epsilon: float = 0.0,
    eigendecomposition_config: EigendecompositionConfig = DefaultEigendecompositionConfig,
    eigenvectors_estimate: Tensor | None = None,
) -> tuple[Tensor, Tensor]:
    """Eigenvalues (ascending) and eigenvectors of symmetric A (+εI when the stability config
    perturbs before the computation)."""
    _require_square(A)
    stability = eigendecomposition_config.rank_deficient_stability_config
    if isinstance(stability, PseudoInverseConfig) and epsilon != 0.0:
        raise ValueError(f"{epsilon=} should be 0.0 when using pseudo-inverse!")
    A_r = _ridge(A, epsilon * getattr(stability, "perturb_before_computation", 0))
    match eigendecomposition_config:
        case EighEigendecompositionConfig(tolerance=tol):
            if tol != 0.0:
                if eigenvectors_estimate is None:
                    raise ValueError(
                        "eigenvectors_estimate should be passed to matrix_eigendecomposition when using tolerance != 0.0."
                    )
                B = eigenvectors_estimate.T @ A_r @ eigenvectors_estimate
                if _nearly_diagonal(B, tol):
                    return B.diag(), eigenvectors_estimate
            return _eigh(
                A_r,
                eigendecomposition_config.retry_double_precision,
                eigendecomposition_config.eigendecomposition_offload_device,
            )
        case QREigendecompositionConfig(max_iterations=iters, tolerance=tol):
            assert eigenvectors_estimate is not None, (
                "eigenvectors_estimate should not be None when QR algorithm is used."
            )
            return _qr_iteration(A_r, eigenvectors_estimate, iters, tol)
        case _:
            raise NotImplementedError(
                f"Eigendecomposition config is not implemented! Specified eigendecomposition config is eigendecomposition_config={eigendecomposition_config}."
            )


# --------------------------------------------------------------------------------------------
# Orthogonalisation (spectral descent / Muon)
# --------------------------------------------------------------------------------------------
def newton_schulz(A: Tensor, num_iterations: int, coefficients: tuple[float, float, float]) -> Tensor:
    """Quintic Newton-Schulz: X ← aX + X(bB + cB²), B = XᵀX, on A/‖A‖_F; wide matrices are
    iterated transposed so that B is the smaller Gram matrix."""
    a, b, c = coefficients
    X = A / torch.clamp(torch.linalg.matrix_norm(A), min=1e-8)
    wide = A.shape[0] < A.shape[1]
    if wide:
        X = X.T
    for _ in range(num_iterations):
        B = X.T @ X
        B = torch.addmm(B, B, B, beta=b, alpha=c)
        X = torch.addmm(X, X, B, beta=a, alpha=1.0)
    return X.T if wide else X


def matrix_orthogonalization(
    A: Tensor,
    orthogonalization_config: OrthogonalizationConfig = DefaultNewtonSchulzOrthogonalizationConfig,
) -> Tensor:
    """Nearest semi-orthogonal matrix to A (polar factor U Vᵀ), exactly by SVD or approximately
    by Newton-Schulz, times ``scale_by_dims_fn(d_in, d_out)``."""
    _require_2d(A)
    scale = orthogonalization_config.scale_by_dims_fn(A.shape[1], A.shape[0])
    match orthogonalization_config:
        case SVDOrthogonalizationConfig(scale_by_nuclear_norm=nuclear):
            U, s, Vh = torch.linalg.svd(A, full_matrices=False)
            out = U @ Vh
            if nuclear:
                out.mul_(s.sum())
        case NewtonSchulzOrthogonalizationConfig(num_iterations=iters, coefficients=coeffs):
            out = newton_schulz(A, iters, coeffs)
        case _:
            raise NotImplementedError(
                f"Orthogonalization config is not implemented! Specified orthogonalization config is orthogonalization_config={orthogonalization_config}."
            )
    return out.mul_(scale) if not out._is_view() else out * scale
