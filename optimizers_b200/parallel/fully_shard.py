"""``fully_shard`` (FSDP2) distributor: every parameter is a DTensor sharded on dim 0; the local
shard is blocked and preconditioned in place.  No optimizer communication; ranks whose shard of
a parameter is empty skip it; block ids carry the rank.

Reference counterpart: ``distributed_shampoo/distributor/shampoo_fully_shard_distributor.py:21-80``.
"""

from __future__ import annotations

from collections.abc import Iterable

import torch
from torch import distributed as dist, Tensor
from torch.distributed.tensor import DTensor

from optimizers_b200.config import PARAMS
from optimizers_b200.parallel.base import Distributor
from optimizers_b200.parallel.block_info import BlockInfo


def local_nonempty_shards(params: Iterable[Tensor], get_grad: bool) -> Iterable[Tensor | None]:
    """Local shards (or the local shards of the gradients) of the DTensor parameters whose local
    shard is not empty."""
    for p in params:
        if p.to_local().numel() == 0:  # type: ignore[attr-defined]
            continue
        if get_grad:
            yield None if p.grad is None else p.grad.to_local()  # type: ignore[union-attr]
        else:
            yield p.to_local()  # type: ignore[attr-defined]


class FullyShardDistributor(Distributor):
    @torch.no_grad()
    def _get_params_or_grads(self, get_grad: bool = False) -> Iterable[Tensor | None]:
        return local_nonempty_shards(self._param_group[PARAMS], get_grad)

    @torch.no_grad()
    def _construct_local_block_info_list(self) -> tuple[BlockInfo, ...]:
        kept = (p for p in self._param_group[PARAMS] if isinstance(p, DTensor) and p.to_local().numel() > 0)
        return self._construct_local_block_info_list_with_params(params=kept, rank=dist.get_rank())
