"""String-to-object resolvers for configuration files and command lines: ``torch_dtype``,
``fsdp_param_strategy``, ``weight_decay_type``.  They are plain functions; when OmegaConf is
installed ``register_resolvers`` also makes them available as ``${torch_dtype:bfloat16}`` etc.

Reference counterpart: ``distributed_shampoo/examples/resolvers.py:16-62``.
"""

from __future__ import annotations

import torch

from optimizers_b200.config import FSDPParamAssignmentStrategy, WeightDecayType


def resolve_torch_dtype(name: str) -> torch.dtype:
    dtype = getattr(torch, name.removeprefix("torch."), None)
    if not isinstance(dtype, torch.dtype):
        raise ValueError(f"Unknown torch dtype: {name}")
    return dtype


def resolve_fsdp_param_strategy(name: str) -> FSDPParamAssignmentStrategy:
    try:
        return FSDPParamAssignmentStrategy[name.upper()]
    except KeyError:
        raise ValueError(f"Unknown FSDPParamAssignmentStrategy: {name}. Valid: {[e.name for e in FSDPParamAssignmentStrategy]}") from None


def resolve_weight_decay_type(name: str) -> WeightDecayType:
    try:
        return WeightDecayType[name.upper()]
    except KeyError:
        raise ValueError(f"Unknown WeightDecayType: {name}. Valid: {[e.name for e in WeightDecayType]}") from None


def register_resolvers() -> bool:
    """Register with OmegaConf if it is installed; returns whether it was."""
    try:
        from omegaconf import OmegaConf
    except ImportError:
        return False
    for key, fn in (
        ("torch_dtype", resolve_torch_dtype),
        ("fsdp_param_strategy", resolve_fsdp_param_strategy),
        ("weight_decay_type", resolve_weight_decay_type),
    ):
        if not OmegaConf.has_resolver(key):
            OmegaConf.register_new_resolver(key, fn)
    return True
