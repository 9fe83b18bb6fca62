"""Lossless ``fully_shard`` distributors: Shampoo on *whole* parameters although the model is
dim-0 sharded, so results equal single-device Shampoo.

REPLICATE    every rank rebuilds every full gradient (``full_tensor()`` per parameter), does all
             the work, and slices its updated full parameters back into its shards.
ROUND_ROBIN  each full parameter has one owner rank (longest-processing-time-first on aligned
             bytes, precomputed by ``split_param_groups``); one all_to_all brings gradient shards
             to the owners, one all_to_all sends the updated parameters back.

The owner keeps full copies of its parameters (``_assigned_full_params``); blocks are views of
these copies.  After a checkpoint load the copies must be re-gathered
(``refresh_assigned_full_params``).

Reference counterpart:
``distributed_shampoo/distributor/shampoo_fully_shard_lossless_distributor.py:35-310``.
"""

from __future__ import annotations

import logging
from collections.abc import Iterable
from typing import Any

import torch
from torch import distributed as dist, Tensor
from torch.distributed import tensor as dtensor

from optimizers_b200.config import (
    DISTRIBUTED_CONFIG,
    FSDPParamAssignmentStrategy,
    FullyShardDistributedConfig,
    OWNER_RANKS,
    PARAMS,
    ShampooRuntimeConfig,
)
from optimizers_b200.parallel.a2a import GatherGradientsContext, RedistributeParamsContext
from optimizers_b200.parallel.base import Distributor
from optimizers_b200.parallel.block_info import BlockInfo
from optimizers_b200.parallel.dist_utils import shampoo_comm_profiler

logger: logging.Logger = logging.getLogger(__name__)


class LosslessShardMixin:
    """Whole-parameter ownership over a shard group; shared by the fully-shard and hybrid-shard
    lossless distributors.  The host class sets ``_shard_dist_group`` before calling
    ``_setup_lossless``."""

    def _setup_lossless(self, param_group: dict[str, Any], shard_group: dist.ProcessGroup) -> None:
        cfg: FullyShardDistributedConfig = param_group[DISTRIBUTED_CONFIG]
        self._param_assignment_strategy = cfg.param_assignment_strategy
        logger.info(f"Shampoo {type(self).__name__} self._param_assignment_strategy={self._param_assignment_strategy}")
        self._shard_dist_group = shard_group
        shard_rank = dist.get_rank(group=shard_group)
        params = param_group[PARAMS]
        if self._param_assignment_strategy == FSDPParamAssignmentStrategy.ROUND_ROBIN:
            owners = param_group.get(OWNER_RANKS)
            assert owners is not None and len(owners) == len(params), (
                "ROUND_ROBIN requires a precomputed OWNER_RANKS map aligned to params (set by split_param_groups); "
                f"got {None if owners is None else len(owners)} for {len(params)} params."
            )
            self._owner_ranks: list[int] | None = list(owners)
            self._assigned_params_mask = tuple(o == shard_rank for o in self._owner_ranks)
            common = dict(
                params=params, assigned_params_mask=self._assigned_params_mask, dist_group=shard_group, owner_ranks=self._owner_ranks
            )
            self._redistribute_ctx: RedistributeParamsContext | None = RedistributeParamsContext(**common)
            self._gather_grads_ctx: GatherGradientsContext | None = GatherGradientsContext(**common)
        else:
            self._owner_ranks = None
            self._assigned_params_mask = (True,) * len(params)
            self._redistribute_ctx = None
            self._gather_grads_ctx = None
        self._param_group = param_group
        self._assigned_full_params: list[Tensor] = self._get_assigned_full_params()

    @torch.no_grad()
    def _get_assigned_full_params(self) -> list[Tensor]:
        if self._gather_grads_ctx is not None:
            return [p for p in self._gather_grads_ctx.gather_params() if p is not None]
        return [p.full_tensor() for p in self._param_group[PARAMS]]

    @torch.no_grad()
    def _get_params_or_grads(self, get_grad: bool = False) -> Iterable[Tensor | None]:
        if not get_grad:
            return (p for p in self._assigned_full_params if isinstance(p, Tensor) and p.numel() > 0)
        name = type(self).__name__
        if self._gather_grads_ctx is not None:
            with shampoo_comm_profiler(f"{name}::gather_gradients_all_to_all"):
                full_grads = self._gather_grads_ctx.gather_gradients()
        else:
            with shampoo_comm_profiler(f"{name}::grad_full_tensors"):
                full_grads = [None if p.grad is None else p.grad.full_tensor() for p in self._param_group[PARAMS]]
        return (
            g
            for g, mine in zip(full_grads, self._assigned_params_mask, strict=True)
            if mine and (g is None or g.numel() > 0)
        )

    def _assigned_nonempty_params(self) -> Iterable[Tensor]:
        return (
            p
            for mine, p in zip(self._assigned_params_mask, self._param_group[PARAMS], strict=True)
            if mine and p.numel() > 0
        )

    @torch.no_grad()
    def _write_back(self) -> None:
        """Bring the updated full parameters back into the local dim-0 shards."""
        if self._redistribute_ctx is not None:
            with shampoo_comm_profiler(f"{type(self).__name__}::_redistribute_ctx.redistribute_and_update_params"):
                self._redistribute_ctx.redistribute_and_update_params(self._assigned_full_params)
        elif self._param_assignment_strategy == FSDPParamAssignmentStrategy.REPLICATE:
            sharded = [p for p in self._param_group[PARAMS] if p.numel() > 0]
            slices = [
                dtensor.distribute_tensor(full, p.device_mesh, p.placements, src_data_rank=None).to_local()
                for p, full in zip(sharded, self._get_params_or_grads(), strict=True)
            ]
            torch._foreach_copy_([p.to_local() for p in sharded], slices)


class FullyShardLosslessDistributor(LosslessShardMixin, Distributor):
    def __init__(self, param_group: dict[str, Any], runtime_config: ShampooRuntimeConfig | None = None) -> None:
        self._group_size: int = dist.get_world_size()
        self._dist_group: dist.ProcessGroup = dist.new_subgroups(group_size=self._group_size)[0]
        self._group_rank: int = dist.get_rank(group=self._dist_group)
        self._setup_lossless(param_group, self._dist_group)
        Distributor.__init__(self, param_group, runtime_config)

    @torch.no_grad()
    def update_params(self, blocked_search_directions: tuple[Tensor, ...], use_masked_tensors: bool = True) -> None:
        Distributor.update_params(self, blocked_search_directions, use_masked_tensors)
        self._write_back()

    @torch.no_grad()
    def _construct_local_block_info_list(self) -> tuple[BlockInfo, ...]:
        return self._construct_local_block_info_list_with_params(params=self._assigned_nonempty_params(), rank=None)

    @torch.no_grad()
    def refresh_assigned_full_params(self) -> None:
        """Re-gather the full copies (their values came from the model, which a checkpoint load has
        just changed) and re-create the block views."""
        self._assigned_full_params = self._get_assigned_full_params()
        self._merge_and_block_parameters()
        self._local_blocked_params = self._global_blocked_params
        self._local_masked_blocked_params = self._local_blocked_params
        self._previous_global_grad_selector = None
