"""Kronecker-factored (Shampoo family) preconditioner lists.

For a block ``G`` of order N with extents ``d_0 … d_{N-1}`` the state is one symmetric factor per
preconditioned dim k,

    F_k ← β2·F_k + w · unfold_k(G) unfold_k(G)ᵀ            (every step)

plus, depending on the variant, what is derived from ``F_k / bc2`` at every refresh
(``perform_amortized_computation``):

* RootInv            ``inv_factor_matrices[k] = (F_k+εI)^(-1/root_k)``; ``P = G ×_k inv_k``
* Eigendecomposed    ``(λ_k, Q_k)``; the inverse root is rebuilt from them when applied
* EigenvalueCorrected (SOAP) ``Q_k`` only, and a running second moment ``V`` of the gradient in
  the eigenbasis: ``P = unproject( project(G) / ((V/bc2)^(1/root) + ε) )``
* KL variants        the Gram matrix of dim k is taken of ``G`` already preconditioned along
  every other dim.

Factors (and inverse roots) are stored as the packed row-major upper triangle when
``use_symmetric_packing``.  A failed refresh keeps the previous value; more than
``num_tolerated_failed_amortized_computations`` consecutive failed refreshes of a block raise.

The classes here hold the state and implement every operation with torch operators.  On a B200
the optimizer drives the same state through the grouped sm_100a kernels
(``optimizers_b200.native_engine``); the methods below then serve as oracle and fallback.

Reference counterpart: ``distributed_shampoo/preconditioner/shampoo_preconditioner_list.py``
(state :106-161, :446-1007; refresh driver :314-443; list :1215-1695; variants :1709-2046).
"""

from __future__ import annotations

import functools

import logging
import math
from collections.abc import Callable, Mapping
from fractions import Fraction
from pathlib import Path
from typing import Any

import torch
from torch import Tensor

from optimizers_b200.config import (
    BaseShampooPreconditionerConfig,
    EigendecompositionConfig,
    PreconditionerValueError,
    SHAMPOO,
)
from optimizers_b200.matrix import functions as mf
from optimizers_b200.parallel.block_info import BlockInfo
from optimizers_b200.preconditioner.base import PreconditionerList, profile_decorator
from optimizers_b200.utils.blocking import (
    compress_list,
    get_dtype_size,
    pack_upper_triangular,
    packed_size,
    unpack_upper_triangular,
)
from optimizers_b200.utils.state import OptimizerModule

logger: logging.Logger = logging.getLogger(__name__)

# Field names of the checkpointed state.
FACTOR_MATRICES = "factor_matrices"
INV_FACTOR_MATRICES = "inv_factor_matrices"
EIGENVECTORS = "factor_matrices_eigenvectors"
EIGENVALUES = "factor_matrices_eigenvalues"
CORRECTED_EIGENVALUES = "corrected_eigenvalues"


@functools.cache
def _packed_diagonal_offsets(d: int, device_type: str, device_index: int | None) -> Tensor:
    """Offsets of the diagonal entries in the packed upper triangle of a d x d matrix, computed on
    the host once per size and device (building them on the device took six launches per factor)."""
    i = torch.arange(d)
    return (i * d - i * (i - 1) // 2).to(torch.device(device_type, device_index))


def _packed_eye(info: BlockInfo, d: int, dtype: torch.dtype, device: torch.device) -> Tensor:
    """Identity in packed form: ones at the offsets of the diagonal entries."""
    t = info.allocate_zeros_tensor(size=(packed_size(d),), dtype=dtype, device=device)
    local = info.get_tensor(t)
    local.index_fill_(0, _packed_diagonal_offsets(d, local.device.type, local.device.index), 1.0)
    return t


class KroneckerFactorsState(OptimizerModule):
    """Checkpointed per-block state.  Which tensor fields exist depends on ``kind``; tuples
    serialise as ``{k: tensor}``; the two non-tensor fields are not checkpointed."""

    def __init__(
        self,
        kind: str,
        info: BlockInfo,
        cfg: BaseShampooPreconditionerConfig,
        dims: tuple[int, ...],
        preconditioned_dims: tuple[int, ...],
    ) -> None:
        device = info.param.device
        packing = cfg.use_symmetric_packing

        def square_zeros(d: int, dtype: torch.dtype) -> Tensor:
            size = (packed_size(d),) if packing else (d, d)
            return info.allocate_zeros_tensor(size=size, dtype=dtype, device=device)

        def square_eye(d: int, dtype: torch.dtype) -> Tensor:
            if packing:
                return _packed_eye(info, d, dtype, device)
            return info.allocate_eye_tensor(n=d, dtype=dtype, device=device)

        self.factor_matrices: tuple[Tensor, ...] = tuple(
            square_zeros(d, cfg.factor_matrix_dtype) for d in preconditioned_dims
        )
        self.factor_matrix_indices: tuple[str, ...] = tuple(
            ".".join((*map(str, info.composable_block_ids), str(k)))
            for k in range(len(preconditioned_dims))
        )
        self.use_symmetric_packing: bool = packing
        if kind == "root_inv":
            self.inv_factor_matrices: tuple[Tensor, ...] = tuple(
                square_eye(d, cfg.inv_factor_matrix_dtype) for d in preconditioned_dims
            )
        elif kind == "eigendecomposed":
            self.factor_matrices_eigenvectors: tuple[Tensor, ...] = tuple(
                info.allocate_eye_tensor(n=d, dtype=cfg.factor_matrix_eigenvectors_dtype, device=device)
                for d in preconditioned_dims
            )
            self.factor_matrices_eigenvalues: tuple[Tensor, ...] = tuple(
                info.allocate_ones_tensor(size=(d,), dtype=cfg.factor_matrix_eigenvalues_dtype, device=device)
                for d in preconditioned_dims
            )
        elif kind == "eigenvalue_corrected":
            self.factor_matrices_eigenvectors = tuple(
                info.allocate_eye_tensor(n=d, dtype=cfg.factor_matrix_eigenvectors_dtype, device=device)
                for d in preconditioned_dims
            )
            self.corrected_eigenvalues: Tensor = info.allocate_zeros_tensor(
                size=tuple(dims), dtype=cfg.corrected_eigenvalues_dtype, device=device
            )
        else:
            raise AssertionError(kind)


def _dump_matrix(factor_matrix_index: str, matrix: Tensor) -> None:
    """Best-effort save of an offending matrix for post-mortem inspection."""
    folder = Path("/tmp").resolve()
    path = folder / f"{factor_matrix_index.replace('.', '_')}.pt"
    try:
        folder.mkdir(exist_ok=True)
        torch.save(matrix, path)
        logger.info(f"Matrix has been saved to {path} for debugging.")
    except Exception as e:
        logger.warning(f"Failed to save matrix to {path}: {str(e)}")


class BlockFactors:
    """Local-tensor view of one block's ``KroneckerFactorsState`` together with what the refresh
    needs (roots, matrix-function config, ε, failure bookkeeping)."""

    def __init__(
        self,
        kind: str,
        state: KroneckerFactorsState,
        get_tensor: Callable[[Tensor], Tensor],
        roots: tuple[float, ...],
        cfg: BaseShampooPreconditionerConfig,
        epsilon: float,
    ) -> None:
        self.kind = kind
        self.use_symmetric_packing = state.use_symmetric_packing
        self.factor_matrix_indices = state.factor_matrix_indices
        self.factor_matrices = tuple(map(get_tensor, state.factor_matrices))
        self.roots = roots
        self.amortized_computation_config = cfg.amortized_computation_config
        self.epsilon = epsilon
        self.num_tolerated_failed_amortized_computations = cfg.num_tolerated_failed_amortized_computations
        self.use_trace_scaling = cfg.use_trace_scaling
        self.trace_scaling_exponent = cfg.trace_scaling_exponent
        self._failed_amortized_computation_counter = 0
        if kind == "root_inv":
            self.inv_factor_matrices = tuple(map(get_tensor, state.inv_factor_matrices))
            assert len(roots) == len(self.factor_matrices) == len(self.inv_factor_matrices)
        elif kind == "eigendecomposed":
            self.factor_matrices_eigenvectors = tuple(map(get_tensor, state.factor_matrices_eigenvectors))
            self.factor_matrices_eigenvalues = tuple(map(get_tensor, state.factor_matrices_eigenvalues))
            assert len(roots) == len(self.factor_matrices) == len(self.factor_matrices_eigenvectors)
        else:
            self.factor_matrices_eigenvectors = tuple(map(get_tensor, state.factor_matrices_eigenvectors))
            self.corrected_eigenvalues = get_tensor(state.corrected_eigenvalues)
            assert len(self.factor_matrices) == len(self.factor_matrices_eigenvectors)
            assert len(roots) == 1

    # -- packing helpers ----------------------------------------------------------------------
    @staticmethod
    def _packed_dim(packed: Tensor) -> int:
        return (math.isqrt(1 + 8 * packed.numel()) - 1) // 2

    def pack(self, m: Tensor) -> Tensor:
        return pack_upper_triangular(m) if self.use_symmetric_packing else m

    def unpack(self, m: Tensor) -> Tensor:
        return unpack_upper_triangular(m, self._packed_dim(m)) if self.use_symmetric_packing else m

    def get_unpacked_factor_matrices(self) -> tuple[Tensor, ...]:
        return tuple(map(self.unpack, self.factor_matrices))

    def get_unpacked_inv_factor_matrices(self) -> tuple[Tensor, ...]:
        return tuple(map(self.unpack, self.inv_factor_matrices))

    # -- refresh ------------------------------------------------------------------------------
    def _compute(self, k: int, A: Tensor) -> tuple[dict[str, Tensor], Exception | None]:
        """Run the configured matrix function on factor k.  Returns the new values keyed by state
        field and the exception if the computation failed (then the old values are returned)."""
        if self.kind == "root_inv":
            old = self.inv_factor_matrices[k]
            try:
                X = mf.matrix_inverse_root(
                    A=A,
                    root=Fraction(self.roots[k]),
                    root_inv_config=self.amortized_computation_config,
                    epsilon=self.epsilon,
                ).to(dtype=old.dtype)
                return {INV_FACTOR_MATRICES: self.pack(X)}, None
            except Exception as exception:
                return {INV_FACTOR_MATRICES: old}, exception
        old_q = self.factor_matrices_eigenvectors[k]
        try:
            lam, Q = mf.matrix_eigendecomposition(
                A=A,
                eigendecomposition_config=self.amortized_computation_config,
                eigenvectors_estimate=old_q.to(dtype=A.dtype),
                epsilon=self.epsilon,
            )
        except Exception as exception:
            out = {EIGENVECTORS: old_q}
            if self.kind == "eigendecomposed":
                out[EIGENVALUES] = self.factor_matrices_eigenvalues[k]
            return out, exception
        if self.kind == "eigendecomposed":
            return {
                EIGENVALUES: lam.to(dtype=self.factor_matrices_eigenvalues[k].dtype),
                EIGENVECTORS: Q.to(dtype=old_q.dtype),
            }, None
        return {EIGENVECTORS: Q.to(dtype=old_q.dtype)}, None

    @profile_decorator
    def amortized_computation(self, bias_correction2: Tensor | float) -> None:
        last_exception: Exception | None = None
        for k, (factor, index) in enumerate(zip(self.factor_matrices, self.factor_matrix_indices, strict=True)):
            A = self.unpack(factor / bias_correction2)
            if self.use_trace_scaling:
                safe_trace = torch.clamp(torch.trace(A), min=self.epsilon)
                A = A * torch.pow(safe_trace, -self.trace_scaling_exponent)
            if not torch.isfinite(A).all():
                raise PreconditionerValueError(
                    f"Encountered nan/inf values in factor matrix {index}! "
                    "To mitigate, check if nan inputs are being passed into the network or nan gradients are being passed to the optimizer. "
                    "Otherwise, in some cases, this may be due to divergence of the algorithm. To mitigate, try decreasing the learning rate or increasing grafting epsilon. "
                    f"For debugging purposes, factor_matrix {index}: "
                    f"torch.min(bias_corrected_factor_matrix)={torch.min(A)}, torch.max(bias_corrected_factor_matrix)={torch.max(A)}, "
                    f"bias_corrected_factor_matrix.isinf().any()={A.isinf().any()}, bias_corrected_factor_matrix.isnan().any()={A.isnan().any()}."
                )
            results, exception = self._compute(k, A)
            if exception:
                last_exception = exception
                _dump_matrix(index, A)
                logger.warning(
                    f"Matrix computation failed for factor matrix {index} with exception={exception!r}. To investigate, check factor matrix before the matrix computation: bias_corrected_factor_matrix={A} Using previous preconditioner and continuing..."
                )
            for field_name, value in results.items():
                if not torch.isfinite(value).all():
                    _dump_matrix(index, A)
                    quantity = field_name.split("_")[-1]
                    raise PreconditionerValueError(
                        f"Encountered nan or inf values in {quantity} of factor matrix {index}! "
                        f"To mitigate, check factor matrix before the matrix computation: bias_corrected_factor_matrix={A}"
                    )
                getattr(self, field_name)[k].copy_(value)
        self.note_refresh_outcome(last_exception)

    def note_refresh_outcome(self, last_exception: Exception | None) -> None:
        """Consecutive-failure counter shared by the torch and the native refresh paths."""
        if last_exception is None:
            self._failed_amortized_computation_counter = 0
            return
        self._failed_amortized_computation_counter += 1
        if self._failed_amortized_computation_counter > self.num_tolerated_failed_amortized_computations:
            raise ValueError(
                f"The number of failed amortized computations for factors {self.factor_matrix_indices} exceeded the allowed tolerance. The last seen exception was {last_exception}."
            ) from last_exception


def mode_k_gram(grad: Tensor, k: int) -> Tensor:
    """Gram matrix of the mode-k unfolding: contracts every dim but k."""
    others = [d for d in range(grad.dim()) if d != k]
    return torch.tensordot(grad, grad, dims=[others, others])


def precondition_grad(
    grad: Tensor,
    preconditioned_dims_selector: tuple[bool, ...],
    preconditioner_list: tuple[Tensor, ...],
    dims: tuple[list[int], list[int]] = ([0], [0]),
) -> Tensor:
    """Multiply ``grad`` along every selected dim by the matching matrix.  Each step contracts
    dim 0 and appends the result dim at the end (or rotates an unselected dim to the end), so
    after N steps the dims are back in order.  ``dims=([0],[1])`` multiplies by the transpose."""
    assert sum(preconditioned_dims_selector) == len(preconditioner_list), (
        f"The number of dimensions to precondition ({sum(preconditioned_dims_selector)}) must match the number of preconditioners ({len(preconditioner_list)})."
    )
    dtypes = {p.dtype for p in preconditioner_list}
    assert len(dtypes) <= 1, f"All preconditioners must have the same dtype, but found: {dtypes}"
    work_dtype = next(iter(dtypes), grad.dtype)
    mats = iter(preconditioner_list)
    out = grad
    for selected in preconditioned_dims_selector:
        if selected:
            out = torch.tensordot(out.to(dtype=work_dtype), next(mats), dims=dims)
        else:
            out = out.permute(*range(1, out.ndim), 0)
    return out.to(dtype=grad.dtype)


class BaseShampooPreconditionerList(PreconditionerList):
    """Shared machinery; subclasses set ``_KIND`` and define which dims are preconditioned, with
    which roots, and how the preconditioner is applied."""

    _KIND = ""

    def __init__(
        self,
        block_list: tuple[Tensor, ...],
        state: Mapping[Tensor, Any],
        block_info_list: tuple[BlockInfo, ...],
        preconditioner_config: BaseShampooPreconditionerConfig,
        beta2: float = 1.0,
        weighting_factor: float = 1.0,
        epsilon: float = 1e-12,
        use_bias_correction: bool = True,
    ) -> None:
        super().__init__(block_list)
        self._preconditioner_config = preconditioner_config
        self._beta2 = beta2
        self._weighting_factor = weighting_factor
        self._epsilon = epsilon
        self._use_bias_correction = use_bias_correction
        self._bias_correction2: Tensor = torch.tensor(1.0)

        selectors = tuple(self._create_preconditioned_dims_selector(dims) for dims in self._dims_list)
        pdims = tuple(compress_list(dims, sel) for dims, sel in zip(self._dims_list, selectors, strict=True))

        factors = []
        for block, info, dims, pd, sel in zip(block_list, block_info_list, self._dims_list, pdims, selectors, strict=True):
            param_index, block_id = info.composable_block_ids
            assert block_id in state[info.param], (
                f"block_index={block_id} not found in state[block_info.param]={state[info.param]}. "
                "The optimizer must create state[param][block_id] before the preconditioners."
            )
            slot = state[info.param][block_id]
            slot[SHAMPOO] = KroneckerFactorsState(self._KIND, info, preconditioner_config, tuple(dims), pd)
            factors.append(
                BlockFactors(
                    self._KIND,
                    slot[SHAMPOO],
                    info.get_tensor,
                    self._get_inverse_roots_from_override(sel),
                    preconditioner_config,
                    epsilon,
                )
            )
            logger.info(
                f"Instantiated Shampoo Preconditioner {param_index}.{block_id} for Parameter {param_index} ({info.param.shape}), Block {block_id} ({block.shape})."
            )

        self._local_kronecker_factors_unwrapped: tuple[BlockFactors, ...] = tuple(factors)
        self._local_order_list: tuple[int, ...] = tuple(b.dim() for b in block_list)
        self._local_preconditioned_dims_selector_list = selectors
        self._masked_kronecker_factors_unwrapped = self._local_kronecker_factors_unwrapped
        self._masked_order_list = self._local_order_list
        self._masked_preconditioned_dims_selector_list = selectors
        self._numel_list = tuple(sum(2 * d * d for d in pd) for pd in pdims)
        factor_bytes = get_dtype_size(preconditioner_config.factor_matrix_dtype)
        self._num_bytes_list = tuple(
            n * (factor_bytes + get_dtype_size(b.dtype)) // 2
            for n, b in zip(self._numel_list, block_list, strict=True)
        )

    # -- variant hooks ------------------------------------------------------------------------
    def _create_preconditioned_dims_selector(self, dims: torch.Size) -> tuple[bool, ...]:
        raise NotImplementedError

    def _get_inverse_roots_from_override(self, preconditioned_dims_selector: tuple[bool, ...]) -> tuple[float, ...]:
        raise NotImplementedError

    def _compute_preconditioned_gradient(self, grad: Tensor, preconditioned_dims_selector: tuple[bool, ...], kronecker_factors: BlockFactors) -> Tensor:
        raise NotImplementedError

    # -- statistics ---------------------------------------------------------------------------
    @profile_decorator
    def _compute_outer_product_list(
        self, grad: Tensor, order: int, preconditioned_dims_selector: tuple[bool, ...], kronecker_factors: BlockFactors
    ) -> tuple[Tensor, ...]:
        return tuple(mode_k_gram(grad, k) for k in compress_list(range(order), preconditioned_dims_selector))

    @profile_decorator
    def _update_factor_matrices(self, masked_grad_list: tuple[Tensor, ...]) -> None:
        for grad, order, sel, kf in zip(
            masked_grad_list,
            self._masked_order_list,
            self._masked_preconditioned_dims_selector_list,
            self._masked_kronecker_factors_unwrapped,
            strict=True,
        ):
            if not kf.factor_matrices:
                continue
            grams = tuple(kf.pack(g) for g in self._compute_outer_product_list(grad, order, sel, kf))
            if self._beta2 != 1.0:
                torch._foreach_mul_(kf.factor_matrices, self._beta2)
            torch._foreach_add_(kf.factor_matrices, grams, alpha=self._weighting_factor)

    def _refresh_bias_correction(self, step: Tensor) -> None:
        if (
            self._use_bias_correction
            and self._beta2 < 1.0
            and not self._preconditioner_config.drop_weighting_factor_on_gsquare
        ):
            self._bias_correction2 = torch.tensor(1.0) - self._beta2**step

    @profile_decorator
    def update_preconditioners(
        self, masked_grad_list: tuple[Tensor, ...], step: Tensor, perform_amortized_computation: bool
    ) -> None:
        self._update_factor_matrices(masked_grad_list)
        self._refresh_bias_correction(step)
        if perform_amortized_computation:
            for kf in self._masked_kronecker_factors_unwrapped:
                kf.amortized_computation(bias_correction2=self._bias_correction2)

    @profile_decorator
    def precondition(self, masked_grad_list: tuple[Tensor, ...]) -> tuple[Tensor, ...]:
        return tuple(
            self._compute_preconditioned_gradient(grad=g, preconditioned_dims_selector=sel, kronecker_factors=kf)
            for g, sel, kf in zip(
                masked_grad_list,
                self._masked_preconditioned_dims_selector_list,
                self._masked_kronecker_factors_unwrapped,
                strict=True,
            )
        )

    @profile_decorator
    def compress_preconditioner_list(self, local_grad_selector: tuple[bool, ...]) -> None:
        self._masked_order_list = compress_list(self._local_order_list, local_grad_selector)
        self._masked_kronecker_factors_unwrapped = compress_list(
            self._local_kronecker_factors_unwrapped, local_grad_selector
        )
        self._masked_preconditioned_dims_selector_list = compress_list(
            self._local_preconditioned_dims_selector_list, local_grad_selector
        )

    # Kept under the reference's name because tests and tools reach for it.
    _precondition_grad = staticmethod(precondition_grad)


class ClassicShampooPreconditionerList(BaseShampooPreconditionerList):
    """Per-dim inverse exponents: default 1/(2·max(order,1)); ``inverse_exponent_override`` may
    replace it per order or per (order, dim); exponent 0 disables the dim."""

    def _get_inverse_exponent(self, dimension: int, order: int) -> float:
        override = self._preconditioner_config.inverse_exponent_override.get(order, {})
        default = 1 / (2 * max(order, 1))
        if isinstance(override, dict):
            return override.get(dimension, default)
        assert isinstance(override, float), (
            f"Expected inverse_exponent_override_on_order to be a float or a dict, but got {type(override)} instead."
        )
        return override

    def _create_preconditioned_dims_selector(self, dims: torch.Size) -> tuple[bool, ...]:
        n = len(dims)
        return tuple(self._get_inverse_exponent(d, n) != 0.0 for d in range(n))

    def _get_inverse_roots_from_override(self, preconditioned_dims_selector: tuple[bool, ...]) -> tuple[float, ...]:
        n = len(preconditioned_dims_selector)
        return tuple(
            1 / self._get_inverse_exponent(k, n) for k, on in enumerate(preconditioned_dims_selector) if on
        )


class RootInvShampooPreconditionerList(ClassicShampooPreconditionerList):
    _KIND = "root_inv"

    def _inverse_roots_of(self, kf: BlockFactors) -> tuple[Tensor, ...]:
        return kf.get_unpacked_inv_factor_matrices()

    def _compute_preconditioned_gradient(self, grad, preconditioned_dims_selector, kronecker_factors) -> Tensor:
        return precondition_grad(grad, preconditioned_dims_selector, self._inverse_roots_of(kronecker_factors))


class EigendecomposedShampooPreconditionerList(ClassicShampooPreconditionerList):
    _KIND = "eigendecomposed"

    def _inverse_roots_of(self, kf: BlockFactors) -> tuple[Tensor, ...]:
        cfg = self._preconditioner_config.amortized_computation_config
        assert isinstance(cfg, EigendecompositionConfig)
        return tuple(
            mf.matrix_inverse_root_from_eigendecomposition(
                L=lam,
                Q=Q,
                root=Fraction(root),
                epsilon=self._epsilon,
                rank_deficient_stability_config=cfg.rank_deficient_stability_config,
            )
            for Q, lam, root in zip(
                kf.factor_matrices_eigenvectors, kf.factor_matrices_eigenvalues, kf.roots, strict=True
            )
        )

    def _compute_preconditioned_gradient(self, grad, preconditioned_dims_selector, kronecker_factors) -> Tensor:
        return precondition_grad(grad, preconditioned_dims_selector, self._inverse_roots_of(kronecker_factors))


class _KLGramMixin:
    """Gram of dim k taken of the gradient preconditioned along all other selected dims."""

    def _compute_outer_product_list(self, grad, order, preconditioned_dims_selector, kronecker_factors):
        inv_roots = self._inverse_roots_of(kronecker_factors)  # type: ignore[attr-defined]
        grams = []
        for pos, k in enumerate(compress_list(range(order), preconditioned_dims_selector)):
            sel = list(preconditioned_dims_selector)
            sel[k] = False
            others = tuple(m for i, m in enumerate(inv_roots) if i != pos)
            grams.append(mode_k_gram(precondition_grad(grad, tuple(sel), others), k))
        return tuple(grams)


class RootInvKLShampooPreconditionerList(_KLGramMixin, RootInvShampooPreconditionerList):
    pass


class EigendecomposedKLShampooPreconditionerList(_KLGramMixin, EigendecomposedShampooPreconditionerList):
    pass


class EigenvalueCorrectedShampooPreconditionerList(BaseShampooPreconditionerList):
    """SOAP: Shampoo's eigenbases with an Adam/AdaGrad second moment kept in the rotated frame."""

    _KIND = "eigenvalue_corrected"

    def _create_preconditioned_dims_selector(self, dims: torch.Size) -> tuple[bool, ...]:
        ignored = self._preconditioner_config.ignored_basis_change_dims.get(len(dims), [])
        return tuple(d not in ignored for d in range(len(dims)))

    def _get_inverse_roots_from_override(self, preconditioned_dims_selector: tuple[bool, ...]) -> tuple[float, ...]:
        order = len(preconditioned_dims_selector)
        return (1 / self._preconditioner_config.inverse_exponent_override.get(order, 1 / 2),)

    @profile_decorator
    def update_preconditioners(self, masked_grad_list, step, perform_amortized_computation) -> None:
        super().update_preconditioners(masked_grad_list, step, perform_amortized_computation)
        for grad, sel, kf in zip(
            masked_grad_list,
            self._masked_preconditioned_dims_selector_list,
            self._masked_kronecker_factors_unwrapped,
            strict=True,
        ):
            rotated = precondition_grad(grad, sel, kf.factor_matrices_eigenvectors)
            if self._beta2 != 1.0:
                kf.corrected_eigenvalues.mul_(self._beta2)
            kf.corrected_eigenvalues.addcmul_(rotated, rotated, value=self._weighting_factor)

    def _compute_preconditioned_gradient(self, grad, preconditioned_dims_selector, kronecker_factors) -> Tensor:
        kf = kronecker_factors
        rotated = precondition_grad(grad.clone(), preconditioned_dims_selector, kf.factor_matrices_eigenvectors)
        rotated.div_(
            kf.corrected_eigenvalues.div(self._bias_correction2).pow_(1 / kf.roots[0]).add_(self._epsilon)
        )
        return precondition_grad(
            rotated, preconditioned_dims_selector, kf.factor_matrices_eigenvectors, dims=([0], [1])
        )
