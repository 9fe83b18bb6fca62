"""Parallelism strategies of the example trainer: how the model is wrapped and which
``DistributedConfig`` the optimizer gets.

Each strategy's ``wrap_model`` returns the wrapped model together with the distributed config
built from it (FSDP1 needs the flat-parameter metadata of the *wrapped* model, the hybrid
strategies need the device mesh).

Reference counterpart: ``distributed_shampoo/examples/parallelism.py:30-212``.
"""

from __future__ import annotations

import abc
from collections.abc import Callable
from dataclasses import dataclass

from torch import nn
from torch.distributed.device_mesh import DeviceMesh

from optimizers_b200.config import DistributedConfig


@dataclass
class WrappedModel:
    model: nn.Module
    distributed_config: DistributedConfig | None = None


class ParallelismStrategy(abc.ABC):
    requires_distributed: bool = False
    requires_device_mesh: bool = False

    def __init__(self, distributed_config: Callable[..., DistributedConfig] | None = None) -> None:
        self.distributed_config = distributed_config

    def _config(self, **kwargs) -> DistributedConfig | None:
        return self.distributed_config(**kwargs) if self.distributed_config else None

    @abc.abstractmethod
    def wrap_model(self, model: nn.Module, local_rank: int, backend: str, device_mesh: DeviceMesh | None = None) -> WrappedModel: ...


class SingleGPUStrategy(ParallelismStrategy):
    def wrap_model(self, model, local_rank, backend, device_mesh=None) -> WrappedModel:
        return WrappedModel(model=model)


class DDPStrategy(ParallelismStrategy):
    requires_distributed = True

    def wrap_model(self, model, local_rank, backend, device_mesh=None) -> WrappedModel:
        from torch.nn.parallel import DistributedDataParallel as DDP

        wrapped = DDP(model, device_ids=[local_rank], output_device=local_rank) if backend == "nccl" else DDP(model)
        return WrappedModel(wrapped, self._config())


class FusedDDPStrategy(ParallelismStrategy):
    """Data parallelism without a gradient all-reduce wrapper: the optimizer's native engine
    reduces the gradients itself (``NativeRuntimeConfig(comm_path="p2p",
    fuse_gradient_reduction=True)``).  Parameters are broadcast once so that ranks start equal."""

    requires_distributed = True

    def wrap_model(self, model, local_rank, backend, device_mesh=None) -> WrappedModel:
        import torch.distributed as dist

        for p in model.parameters():
            dist.broadcast(p.data, src=0)
        return WrappedModel(model, self._config())


class FSDPStrategy(ParallelismStrategy):
    requires_distributed = True

    def wrap_model(self, model, local_rank, backend, device_mesh=None) -> WrappedModel:
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP

        from optimizers_b200.parallel.fsdp_utils import compile_fsdp_parameter_metadata

        wrapped = FSDP(model, use_orig_params=True)
        return WrappedModel(wrapped, self._config(param_to_metadata=compile_fsdp_parameter_metadata(wrapped)))


class HSDPStrategy(ParallelismStrategy):
    requires_distributed = True
    requires_device_mesh = True

    def wrap_model(self, model, local_rank, backend, device_mesh=None) -> WrappedModel:
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, ShardingStrategy

        from optimizers_b200.parallel.fsdp_utils import compile_fsdp_parameter_metadata

        assert device_mesh is not None
        wrapped = FSDP(model, device_mesh=device_mesh, sharding_strategy=ShardingStrategy.HYBRID_SHARD, use_orig_params=True)
        return WrappedModel(
            wrapped, self._config(param_to_metadata=compile_fsdp_parameter_metadata(wrapped), device_mesh=device_mesh)
        )


class FullyShardStrategy(ParallelismStrategy):
    requires_distributed = True

    def wrap_model(self, model, local_rank, backend, device_mesh=None) -> WrappedModel:
        from torch.distributed.fsdp import fully_shard

        return WrappedModel(fully_shard(model), self._config())


class HybridShardStrategy(ParallelismStrategy):
    requires_distributed = True
    requires_device_mesh = True

    def wrap_model(self, model, local_rank, backend, device_mesh=None) -> WrappedModel:
        from torch.distributed.fsdp import fully_shard

        assert device_mesh is not None
        return WrappedModel(fully_shard(model, mesh=device_mesh), self._config(device_mesh=device_mesh))


STRATEGIES: dict[str, type[ParallelismStrategy]] = {
    "none": SingleGPUStrategy,
    "ddp": DDPStrategy,
    "ddp_fused": FusedDDPStrategy,
    "fsdp": FSDPStrategy,
    "hsdp": HSDPStrategy,
    "fully_shard": FullyShardStrategy,
    "hybrid_shard": HybridShardStrategy,
}
