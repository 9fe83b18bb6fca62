"""Distributor interface and the single-device distributor.

A distributor decides, for one parameter group, how parameters are cut into blocks, which blocks
this rank works on, and how computed search directions reach the parameters (locally, or through
a collective).  Blocks are detached *views* of the parameters, so updating a block updates the
model in place; gradients are blocked the same way every step without copies.

Three selectors describe the blocks, all in global block order:

* ``_global_grad_selector``  -- the block's parameter received a non-empty gradient this step
* ``_distributor_selector``  -- the block is assigned to this rank
* ``local_grad_selector``    -- the first restricted to the second (one bit per local block)

Reference counterpart: ``distributed_shampoo/distributor/shampoo_distributor.py:34-430``.
"""

from __future__ import annotations

import abc
from collections.abc import Iterable
from typing import Any

import torch
from torch import Tensor

from optimizers_b200.config import (
    DISTRIBUTED_CONFIG,
    MAX_PRECONDITIONER_DIM,
    PARAMS,
    ShampooRuntimeConfig,
)
from optimizers_b200.parallel.block_info import BlockInfo
from optimizers_b200.utils.blocking import (
    compress_list,
    generate_pairwise_indices,
    merge_small_dims,
    multi_dim_split,
)


class DistributorInterface(abc.ABC):
    def __init__(self, param_group: dict[str, Any], runtime_config: ShampooRuntimeConfig | None = None) -> None:
        self._param_group = param_group
        self._runtime_config = runtime_config if runtime_config is not None else ShampooRuntimeConfig()
        self._merge_and_block_parameters()
        self._global_grad_selector: tuple[bool, ...] = (True,) * len(self._global_blocked_params)
        self._previous_global_grad_selector: tuple[bool, ...] | None = None
        # Set by subclasses:
        self._distributor_selector: tuple[bool, ...]
        self._local_grad_selector: tuple[bool, ...]
        self._local_blocked_params: tuple[Tensor, ...]
        self._local_masked_blocked_params: tuple[Tensor, ...]
        self._local_block_info_list: tuple[BlockInfo, ...]

    # -- API used by the optimizer -------------------------------------------------------------
    @abc.abstractmethod
    def update_params(self, blocked_search_directions: tuple[Tensor, ...], use_masked_tensors: bool = True) -> None:
        """Add the search directions to the parameters; ``use_masked_tensors=False`` addresses
        every local block instead of only those with a gradient."""

    @abc.abstractmethod
    def merge_and_block_gradients(self) -> tuple[Tensor, ...]:
        """Blocked gradients of the local blocks that have one; refreshes the selectors."""

    @property
    def local_grad_selector(self) -> tuple[bool, ...]:
        return self._local_grad_selector

    @property
    def local_blocked_params(self) -> tuple[Tensor, ...]:
        return self._local_blocked_params

    @property
    def local_masked_blocked_params(self) -> tuple[Tensor, ...]:
        return self._local_masked_blocked_params

    @property
    def local_block_info_list(self) -> tuple[BlockInfo, ...]:
        return self._local_block_info_list

    # -- blocking ------------------------------------------------------------------------------
    def _construct_composable_block_ids(
        self, param_index: int, block_index: int, rank: int | None = None
    ) -> tuple[int, str]:
        """``(param_index, "block_i")`` or ``(param_index, "rank_r-block_i")``."""
        label = f"block_{block_index}"
        return param_index, (label if rank is None else f"rank_{rank}-{label}")

    @torch.no_grad()
    def _get_params_or_grads(self, get_grad: bool = False) -> Iterable[Tensor | None]:
        params = self._param_group[PARAMS]
        return (p.grad for p in params) if get_grad else params

    def _blocks_of(self, tensor: Tensor) -> tuple[Tensor, ...]:
        threshold = self._param_group[MAX_PRECONDITIONER_DIM]
        target = self._param_group[DISTRIBUTED_CONFIG].target_parameter_dimensionality
        merged_shape = merge_small_dims(tuple(tensor.size()), threshold, target)
        return multi_dim_split(tensor.view(merged_shape), threshold)

    @torch.no_grad()
    def _merge_and_block_with_params(self, params: Iterable[Tensor]) -> tuple[list[Tensor], list[int]]:
        blocks: list[Tensor] = []
        counts: list[int] = []
        for p in params:
            pieces = self._blocks_of(p)
            blocks.extend(piece.detach() for piece in pieces)
            counts.append(len(pieces))
        return blocks, counts

    def _merge_and_block_parameters(self) -> None:
        blocks, counts = self._merge_and_block_with_params(self._get_params_or_grads())
        self._global_blocked_params: tuple[Tensor, ...] = tuple(blocks)
        self._global_num_blocks_per_param: tuple[int, ...] = tuple(counts)

    def _merge_and_block_gradients(self) -> tuple[Tensor, ...]:
        local_grads: list[Tensor] = []
        selector: list[bool] = []
        for grad, count, (lo, hi) in zip(
            self._get_params_or_grads(get_grad=True),
            self._global_num_blocks_per_param,
            generate_pairwise_indices(self._global_num_blocks_per_param),
            strict=True,
        ):
            mine = self._distributor_selector[lo:hi]
            usable = grad is not None and grad.numel() > 0
            selector.extend([usable] * count)
            if not usable or not any(mine):
                continue
            if self._runtime_config.eager_nan_check:
                assert torch.isfinite(grad).all(), (
                    f"Encountered gradient containing NaN/Inf in parameter with shape {grad.shape}. Check your model for numerical instability or consider gradient clipping."
                )
            local_grads.extend(compress_list(self._blocks_of(grad), mine))
        self._global_grad_selector = tuple(selector)
        return tuple(local_grads)

    def _refresh_local_selection(self) -> None:
        """Recompute the local selector and the masked parameter list after the global gradient
        selector changed."""
        if self._previous_global_grad_selector == self._global_grad_selector:
            return
        self._previous_global_grad_selector = self._global_grad_selector
        self._local_grad_selector = compress_list(self._global_grad_selector, self._distributor_selector)
        self._local_masked_blocked_params = compress_list(self._local_blocked_params, self._local_grad_selector)

    @torch.no_grad()
    def _construct_local_block_info_list_with_params(
        self, params: Iterable[Tensor], rank: int | None = None
    ) -> tuple[BlockInfo, ...]:
        return tuple(
            BlockInfo(
                param=p,
                composable_block_ids=self._construct_composable_block_ids(param_index, b, rank),
            )
            for (param_index, p), count in zip(enumerate(params), self._global_num_blocks_per_param, strict=True)
            for b in range(count)
        )


class Distributor(DistributorInterface):
    """Single device: every block is local and the update is a fused add."""

    def __init__(self, param_group: dict[str, Any], runtime_config: ShampooRuntimeConfig | None = None) -> None:
        super().__init__(param_group, runtime_config)
        n = len(self._global_blocked_params)
        self._local_grad_selector = (True,) * n
        self._distributor_selector = self._local_grad_selector
        self._local_blocked_params = self._global_blocked_params
        self._local_masked_blocked_params = self._local_blocked_params
        self._local_block_info_list = self._construct_local_block_info_list()

    @torch.no_grad()
    def _construct_local_block_info_list(self) -> tuple[BlockInfo, ...]:
        return self._construct_local_block_info_list_with_params(self._get_params_or_grads())

    @torch.no_grad()
    def update_params(self, blocked_search_directions: tuple[Tensor, ...], use_masked_tensors: bool = True) -> None:
        targets = self._local_masked_blocked_params if use_masked_tensors else self._local_blocked_params
        assert len(blocked_search_directions) == len(targets), (
            f"Expected len(blocked_search_directions)={len(blocked_search_directions)} to be equal to len(target_params)={len(targets)}."
        )
        if blocked_search_directions:
            torch._foreach_add_(targets, blocked_search_directions)

    def merge_and_block_gradients(self) -> tuple[Tensor, ...]:
        grads = self._merge_and_block_gradients()
        self._refresh_local_selection()
        return grads
