"""Hybrid-shard (FSDP2 ``fully_shard`` on a 2-D mesh) distributor: local dim-0 shards are blocked
like the fully-shard distributor does, and the ranks holding the same shard (the replicate mesh
dimension) share the optimizer work of it ZeRO-1 style with one all-gather per step, like the
DDP distributor.

Reference counterpart: ``distributed_shampoo/distributor/shampoo_hybrid_shard_distributor.py:44-596``.
"""

from __future__ import annotations

from collections.abc import Iterable
from functools import partial
from typing import Any

import torch
from torch import Tensor
from torch.distributed.tensor import DTensor

from optimizers_b200.config import DISTRIBUTED_CONFIG, HybridShardDistributedConfig, PARAMS, ShampooRuntimeConfig
from optimizers_b200.parallel.block_info import DTensorBlockInfo
from optimizers_b200.parallel.ddp import DDPDistributor
from optimizers_b200.parallel.fully_shard import local_nonempty_shards
from optimizers_b200.parallel.hsdp import resolve_replicate_group
from optimizers_b200.utils.blocking import generate_pairwise_indices


class HybridShardDistributor(DDPDistributor):
    def __init__(self, param_group: dict[str, Any], runtime_config: ShampooRuntimeConfig | None = None) -> None:
        cfg: HybridShardDistributedConfig = param_group[DISTRIBUTED_CONFIG]
        self._hybrid_shard_device_mesh = cfg.device_mesh
        super().__init__(param_group, runtime_config)

    def _resolve_group(self, cfg: HybridShardDistributedConfig, dist_group: Any) -> None:
        resolve_replicate_group(self, cfg, self._hybrid_shard_device_mesh)
        self._block_id_rank = self._get_composable_block_id_rank()

    def _get_composable_block_id_rank(self) -> int | None:
        """Position in the shard dimension: different shard ranks hold different pieces of the same
        parameter, so their block ids must differ."""
        return self._hybrid_shard_device_mesh.get_local_rank(1)

    @torch.no_grad()
    def _get_params_or_grads(self, get_grad: bool = False) -> Iterable[Tensor | None]:
        return local_nonempty_shards(self._param_group[PARAMS], get_grad)

    def _block_info_params(self) -> Iterable[Tensor]:
        return (p for p in self._param_group[PARAMS] if isinstance(p, DTensor) and p.to_local().numel() > 0)

    @torch.no_grad()
    def _construct_local_block_info_list(
        self, group_source_ranks: tuple[int, ...], group_rank: int
    ) -> tuple[DTensorBlockInfo, ...]:
        infos = []
        for (param_index, p), (lo, hi) in zip(
            enumerate(self._block_info_params()),
            generate_pairwise_indices(self._global_num_blocks_per_param),
            strict=True,
        ):
            for block_index, owner in enumerate(group_source_ranks[lo:hi]):
                if owner != group_rank:
                    continue
                infos.append(
                    DTensorBlockInfo(
                        param=p,
                        composable_block_ids=self._construct_composable_block_ids(
                            param_index, block_index, self._block_id_rank
                        ),
                        allocate_zeros_tensor=partial(self._allocate_zeros_distributed_tensor, group_source_rank=owner),
                    )
                )
        return tuple(infos)

    def _allocate_global_buffer(self, nbytes: int) -> Tensor:
        return torch.zeros(nbytes, dtype=torch.int8, device=self._param_group[PARAMS][0].device)
