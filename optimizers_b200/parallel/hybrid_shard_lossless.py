"""Lossless hybrid-shard distributor: whole-parameter ownership along the shard dimension
(REPLICATE or ROUND_ROBIN, see ``fully_shard_lossless``) combined with ZeRO-1 style work sharing
and an all-gather along the replicate dimension.

Every instance builds a private device mesh (unique dimension names) so that its collectives run
on communicators of its own; sub-groups of one optimizer can then overlap on separate streams
without ordering hazards between their collectives.

Reference counterpart:
``distributed_shampoo/distributor/shampoo_hybrid_shard_lossless_distributor.py:42-360``.
"""

from __future__ import annotations

import copy
import itertools
from collections.abc import Iterable
from typing import Any

import torch
from torch import Tensor
from torch.distributed.device_mesh import init_device_mesh

from optimizers_b200.config import DISTRIBUTED_CONFIG, HybridShardDistributedConfig, ShampooRuntimeConfig
from optimizers_b200.parallel.fully_shard_lossless import LosslessShardMixin
from optimizers_b200.parallel.hybrid_shard import HybridShardDistributor
from optimizers_b200.utils.blocking import compress_list


class HybridShardLosslessDistributor(LosslessShardMixin, HybridShardDistributor):
    _instance_counter = itertools.count()

    def __init__(self, param_group: dict[str, Any], runtime_config: ShampooRuntimeConfig | None = None) -> None:
        cfg: HybridShardDistributedConfig = param_group[DISTRIBUTED_CONFIG]
        idx = next(HybridShardLosslessDistributor._instance_counter)
        mesh = cfg.device_mesh
        names = mesh.mesh_dim_names
        assert names is not None, "DeviceMesh must have mesh_dim_names"
        self._device_mesh = init_device_mesh(
            mesh.device_type, tuple(mesh.mesh.shape), mesh_dim_names=tuple(f"{idx}_{n}" for n in names)
        )
        cfg = copy.copy(cfg)
        cfg.device_mesh = self._device_mesh
        param_group[DISTRIBUTED_CONFIG] = cfg
        self._shard_group_size: int = self._device_mesh.size(1)
        shard_group = self._device_mesh.get_group(mesh_dim=1)
        self._shard_group_rank: int = torch.distributed.get_rank(shard_group)
        self._setup_lossless(param_group, shard_group)
        HybridShardDistributor.__init__(self, param_group, runtime_config)

    def _get_composable_block_id_rank(self) -> int | None:
        return None  # blocks are cut from whole parameters: the same on every shard rank

    def _get_params_or_grads(self, get_grad: bool = False) -> Iterable[Tensor | None]:
        return LosslessShardMixin._get_params_or_grads(self, get_grad)

    def _block_info_params(self) -> Iterable[Tensor]:
        return self._assigned_nonempty_params()

    @torch.no_grad()
    def update_params(self, blocked_search_directions: tuple[Tensor, ...], use_masked_tensors: bool = True) -> None:
        HybridShardDistributor.update_params(self, blocked_search_directions, use_masked_tensors)
        self._write_back()

    @torch.no_grad()
    def refresh_assigned_full_params(self) -> None:
        self._assigned_full_params = self._get_assigned_full_params()
        self._merge_and_block_parameters()
        self._local_blocked_params = compress_list(self._global_blocked_params, self._distributor_selector)
        self._local_masked_blocked_params = self._local_blocked_params
        self._global_masked_blocked_params = self._global_blocked_params
        # The gather-buffer views keep their layout; only the parameter views changed.
        self._global_masked_dist_blocked_buffers = self._global_dist_blocked_buffers
        self._local_masked_dist_blocked_buffers = self._local_dist_blocked_buffers
        self._previous_global_grad_selector = None
