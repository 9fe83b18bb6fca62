"""HSDP1 (FSDP1 ``HYBRID_SHARD``) distributor.

Within the shard dimension of the 2-D device mesh each rank holds FSDP1 flat-parameter slices,
blocked like the FSDP distributor does.  Ranks at the same shard position (the replicate
dimension, size R) hold identical slices; they are cut into groups of
``num_trainers_per_group`` that share the optimizer work of those slices ZeRO-1 style, with one
all-gather along that group per step, exactly like the DDP distributor.

Reference counterpart: ``distributed_shampoo/distributor/shampoo_hsdp_distributor.py:45-886``.
"""

from __future__ import annotations

import logging
from typing import Any

from torch import distributed as dist

from optimizers_b200.config import DISTRIBUTED_CONFIG, HSDPDistributedConfig, ShampooRuntimeConfig
from optimizers_b200.parallel.ddp import DDPDistributor
from optimizers_b200.parallel.dist_utils import batched, create_hybrid_shard_process_groups
from optimizers_b200.parallel.fsdp import FlatShardBlocking

logger: logging.Logger = logging.getLogger(__name__)


def resolve_replicate_group(distributor: Any, cfg: Any, device_mesh: Any) -> None:
    """Group set-up shared by the HSDP and hybrid-shard distributors: the communication group is
    a sub-group of the mesh's replicate dimension."""
    if not dist.is_initialized():
        raise RuntimeError(f"{type(distributor).__name__} needs torch.distributed to be initialized!")
    replicated = device_mesh.size(0)
    n = cfg.num_trainers_per_group
    if not (1 <= n <= replicated or n == -1):
        raise ValueError(
            f"Invalid number of trainers per group: {n}. Must be between [1, {replicated}] or set to -1."
        )
    if n == -1:
        logger.info(
            f"Note that distributed_config.num_trainers_per_group={n}! Defaulting to replicated group size {replicated}."
        )
    elif replicated % n != 0:
        raise ValueError(
            f"distributed_config.num_trainers_per_group={n} must divide self._replicated_group_size={replicated}!"
        )
    distributor._replicated_group_size = replicated
    distributor._global_size = replicated
    distributor._group_size = n if n != -1 else replicated
    distributor._dist_group_size = distributor._group_size
    distributor._dist_group = create_hybrid_shard_process_groups(device_mesh, distributor._group_size)
    distributor._comms_dist_group = distributor._dist_group
    same_shard_ranks = dist.get_process_group_ranks(device_mesh.get_group(0))
    distributor._owner_mesh_rows = tuple(batched(same_shard_ranks, distributor._group_size))
    distributor._block_id_rank = device_mesh.get_local_rank(1)


class HSDPDistributor(FlatShardBlocking, DDPDistributor):
    def __init__(self, param_group: dict[str, Any], runtime_config: ShampooRuntimeConfig | None = None) -> None:
        cfg: HSDPDistributedConfig = param_group[DISTRIBUTED_CONFIG]
        self._param_to_metadata = cfg.param_to_metadata
        self._hsdp_device_mesh = cfg.device_mesh
        self._global_num_splits_per_param: tuple[int, ...] = ()
        self._global_num_blocks_per_split_param: tuple[int, ...] = ()
        super().__init__(param_group, runtime_config)

    def _resolve_group(self, cfg: HSDPDistributedConfig, dist_group: Any) -> None:
        resolve_replicate_group(self, cfg, self._hsdp_device_mesh)

    def _get_params_or_grads(self, get_grad: bool = False):
        params = self._param_group["params"]
        return (p.grad for p in params) if get_grad else params
