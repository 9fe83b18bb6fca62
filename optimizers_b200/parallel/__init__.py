"""Distributors: how blocks are shared between ranks and how updates reach the parameters.

Distributor classes are resolved lazily so that importing the package does not import
``torch.distributed`` sub-packages that a single-device user never needs.
"""

from __future__ import annotations

import importlib

from optimizers_b200.parallel.base import Distributor, DistributorInterface
from optimizers_b200.parallel.block_info import BlockInfo, DTensorBlockInfo

_LAZY = {
    "DDPDistributor": "optimizers_b200.parallel.ddp",
    "FSDPDistributor": "optimizers_b200.parallel.fsdp",
    "HSDPDistributor": "optimizers_b200.parallel.hsdp",
    "FullyShardDistributor": "optimizers_b200.parallel.fully_shard",
    "FullyShardLosslessDistributor": "optimizers_b200.parallel.fully_shard_lossless",
    "HybridShardDistributor": "optimizers_b200.parallel.hybrid_shard",
    "HybridShardLosslessDistributor": "optimizers_b200.parallel.hybrid_shard_lossless",
}


def __getattr__(name: str):
    if name in _LAZY:
        return getattr(importlib.import_module(_LAZY[name]), name)
    raise AttributeError(name)


__all__ = ["BlockInfo", "DTensorBlockInfo", "Distributor", "DistributorInterface", *_LAZY]
