"""Stateless and diagonal preconditioner lists: SGD (identity), AdaGrad/RMSprop/Adam (diagonal
second moment), sign descent and spectral descent (Muon-style orthogonalised update).

Reference counterparts: ``distributed_shampoo/preconditioner/sgd_preconditioner_list.py:14-42``,
``adagrad_preconditioner_list.py:33-170``, ``sign_descent_preconditioner_list.py:19-55``,
``spectral_descent_preconditioner_list.py:19-68``.
"""

from __future__ import annotations

import logging
from collections.abc import Mapping
from typing import Any

import torch
from torch import Tensor

from optimizers_b200.config import (
    ADAGRAD,
    SignDescentPreconditionerConfig,
    SpectralDescentPreconditionerConfig,
)
from optimizers_b200.matrix.functions import matrix_orthogonalization
from optimizers_b200.parallel.block_info import BlockInfo
from optimizers_b200.preconditioner.base import PreconditionerList, profile_decorator
from optimizers_b200.utils.blocking import compress_list

logger: logging.Logger = logging.getLogger(__name__)


class SGDPreconditionerList(PreconditionerList):
    """P = G."""

    def update_preconditioners(self, masked_grad_list, step, perform_amortized_computation=False) -> None:
        return

    def precondition(self, masked_grad_list: tuple[Tensor, ...]) -> tuple[Tensor, ...]:
        return masked_grad_list

    def compress_preconditioner_list(self, local_grad_selector: tuple[bool, ...]) -> None:
        return


class AdagradPreconditionerList(PreconditionerList):
    """V ← β2·V + w·G²;  P = G / (sqrt(V / bc2) + ε), with bc2 = 1 - β2^t when bias correction
    applies.  β2 = 1, w = 1 is AdaGrad; β2 < 1, w = 1-β2 is RMSprop (no bias correction) or Adam.

    State: one tensor ``"adagrad"`` of the block's shape and dtype per block.
    """

    def __init__(
        self,
        block_list: tuple[Tensor, ...],
        state: Mapping[Tensor, Any],
        block_info_list: tuple[BlockInfo, ...],
        beta2: float = 1.0,
        weighting_factor: float = 1.0,
        epsilon: float = 1e-10,
        use_bias_correction: bool = True,
    ) -> None:
        super().__init__(block_list)
        self._beta2 = beta2
        self._weighting_factor = weighting_factor
        self._epsilon = epsilon
        self._use_bias_correction = use_bias_correction
        self._bias_correction2: Tensor = torch.tensor(1.0)

        moments = []
        for block, info in zip(block_list, block_info_list, strict=True):
            param_index, block_id = info.composable_block_ids
            assert block_id in state[info.param], (
                f"block_index={block_id} not found in state[block_info.param]={state[info.param]}. "
                "The optimizer must create state[param][block_id] before the preconditioners."
            )
            slot = state[info.param][block_id]
            slot[ADAGRAD] = info.allocate_zeros_tensor(
                size=block.size(), dtype=block.dtype, device=block.device
            )
            moments.append(info.get_tensor(slot[ADAGRAD]))
            logger.info(
                f"Instantiated Adagrad Preconditioner {param_index}.{block_id} ({slot[ADAGRAD].shape} with dtype {slot[ADAGRAD].dtype}) "
                f"for Parameter {param_index} ({info.param.shape}), Block {block_id} ({block.shape})."
            )
        self._local_preconditioner_list: tuple[Tensor, ...] = tuple(moments)
        self._masked_preconditioner_list = self._local_preconditioner_list
        self._numel_list = tuple(m.numel() for m in moments)
        self._num_bytes_list = tuple(m.numel() * m.element_size() for m in moments)

    @profile_decorator
    def update_preconditioners(self, masked_grad_list, step, perform_amortized_computation=False) -> None:
        if self._beta2 != 1.0:
            torch._foreach_mul_(self._masked_preconditioner_list, self._beta2)
        torch._foreach_addcmul_(
            self._masked_preconditioner_list, masked_grad_list, masked_grad_list, value=self._weighting_factor
        )
        if self._use_bias_correction and self._beta2 < 1.0:
            self._bias_correction2 = torch.tensor(1.0) - self._beta2**step

    @profile_decorator
    def precondition(self, masked_grad_list: tuple[Tensor, ...]) -> tuple[Tensor, ...]:
        denom = torch._foreach_div(self._masked_preconditioner_list, self._bias_correction2)
        torch._foreach_sqrt_(denom)
        torch._foreach_add_(denom, self._epsilon)
        return tuple(torch._foreach_div(masked_grad_list, denom))

    @profile_decorator
    def compress_preconditioner_list(self, local_grad_selector: tuple[bool, ...]) -> None:
        self._masked_preconditioner_list = compress_list(
            self._local_preconditioner_list, local_grad_selector
        )


class SignDescentPreconditionerList(PreconditionerList):
    """P = sign(G) · scale_fn(G)."""

    def __init__(self, block_list: tuple[Tensor, ...], preconditioner_config: SignDescentPreconditionerConfig) -> None:
        super().__init__(block_list)
        self._preconditioner_config = preconditioner_config

    @profile_decorator
    def update_preconditioners(self, masked_grad_list, step, perform_amortized_computation=False) -> None:
        return

    @profile_decorator
    def precondition(self, masked_grad_list: tuple[Tensor, ...]) -> tuple[Tensor, ...]:
        scale_fn = self._preconditioner_config.scale_fn
        return tuple(torch.sign(g).mul_(scale_fn(g)) for g in masked_grad_list)

    def compress_preconditioner_list(self, local_grad_selector: tuple[bool, ...]) -> None:
        return


class SpectralDescentPreconditionerList(PreconditionerList):
    """P = orthogonalise(G) for 2-D blocks only."""

    def __init__(
        self,
        block_list: tuple[Tensor, ...],
        preconditioner_config: SpectralDescentPreconditionerConfig,
        native_gemm_mode: str | None = None,
    ) -> None:
        if any(b.dim() != 2 for b in block_list):
            raise ValueError(
                "Spectral descent can only be used for 2D parameters, or parameters that have been reshaped to 2D. "
                "To guarantee that all >2D parameters are reshaped to 2D, set max_preconditioner_dim=math.inf and distributed_config.target_parameter_dimensionality=2."
            )
        super().__init__(block_list)
        self._preconditioner_config = preconditioner_config
        # "tf32x3" / "tf32": run Newton-Schulz for all blocks together on the grouped tensor-core
        # GEMM when the gradients are fp32 tensors on an sm_100 device; None: per-block torch path.
        self._native_gemm_mode = native_gemm_mode
        self._batched: dict[tuple[tuple[int, int], ...], object] = {}

    @profile_decorator
    def update_preconditioners(self, masked_grad_list, step, perform_amortized_computation=False) -> None:
        return

    def _batched_newton_schulz(self, grads: tuple[Tensor, ...], cfg) -> tuple[Tensor, ...] | None:
        from optimizers_b200.config import NewtonSchulzOrthogonalizationConfig

        if (
            self._native_gemm_mode is None or not grads or not isinstance(cfg, NewtonSchulzOrthogonalizationConfig)
            or any(not g.is_cuda or g.dtype != torch.float32 for g in grads)
            or torch.cuda.get_device_capability(grads[0].device)[0] != 10
        ):
            return None
        from optimizers_b200.matrix.batched import BatchedNewtonSchulz
        from optimizers_b200.ops import build

        key = tuple((g.shape[0], g.shape[1]) for g in grads)
        runner = self._batched.get(key)
        if runner is None:
            self._batched.clear()  # one live set of buffers: the selection changes rarely
            runner = BatchedNewtonSchulz(build.load(), list(key), grads[0].device, split=self._native_gemm_mode == "tf32x3")
            self._batched[key] = runner
        out = runner(list(grads), cfg.num_iterations, cfg.coefficients)
        scales = [cfg.scale_by_dims_fn(g.shape[1], g.shape[0]) for g in grads]
        if any(sc != 1.0 for sc in scales):
            torch._foreach_mul_(out, scales)
        return tuple(out)

    @profile_decorator
    def precondition(self, masked_grad_list: tuple[Tensor, ...]) -> tuple[Tensor, ...]:
        cfg = self._preconditioner_config.orthogonalization_config
        native = self._batched_newton_schulz(masked_grad_list, cfg)
        if native is not None:
            return native
        return tuple(matrix_orthogonalization(g, orthogonalization_config=cfg) for g in masked_grad_list)

    def compress_preconditioner_list(self, local_grad_selector: tuple[bool, ...]) -> None:
        return
