"""Helpers for models wrapped by FSDP1 (flat parameters) or ``fully_shard`` (per-parameter
DTensors): per-parameter shard metadata, and partitioning of parameter collections into
FSDP-sharded, hybrid-sharded and unsharded subsets.

Reference counterpart: ``distributed_shampoo/distributor/shampoo_fsdp_utils.py:20-250``.
"""

from __future__ import annotations

import itertools
from collections.abc import Callable, Iterable

import torch
from torch.distributed.fsdp import FullyShardedDataParallel as FSDP, ShardingStrategy
from torch.distributed.tensor import DTensor
from torch.optim.optimizer import ParamsT

from optimizers_b200.config import FSDPParameterMetadata


def compile_fsdp_parameter_metadata(module: torch.nn.Module) -> dict[torch.nn.Parameter, FSDPParameterMetadata]:
    """For every original parameter of an FSDP1 model (``use_orig_params=True``): its name, full
    shape and the half-open index range of it that this rank's flat shard holds.  Reads FSDP's
    flat-parameter bookkeeping (``_fqns``, ``_shapes``, ``_numels``, ``_shard_param_infos``)."""
    out: dict[torch.nn.Parameter, FSDPParameterMetadata] = {}
    for fsdp_module in FSDP.fsdp_modules(module):
        flat = fsdp_module._flat_param
        if flat is None:
            continue
        assert flat._params is not None, (
            "flat_param._params should not be None! Set the value of `use_orig_params` in FSDP module to True "
            "would populate flat_param._params."
        )
        strategy = fsdp_module.sharding_strategy
        for p, fqn, shape, numel, info in zip(
            flat._params, flat._fqns, flat._shapes, flat._numels, flat._shard_param_infos, strict=True
        ):
            start = info.intra_param_start_idx or 0
            end = info.intra_param_end_idx + 1 if info.intra_param_end_idx is not None else 0
            out[p] = FSDPParameterMetadata(
                fqn=fqn, shape=shape, numel=numel, start_idx=start, end_idx=end, sharding_strategy=strategy
            )
    return out


def _partition_params(
    params: ParamsT, fsdp_criteria: Callable[[torch.Tensor], bool], hsdp_criteria: Callable[[torch.Tensor], bool]
) -> tuple[ParamsT, ParamsT, ParamsT]:
    """Split ``params`` (tensors, param-group dicts, or ``(name, tensor)`` pairs) three ways while
    keeping the container kind."""

    def neither(p: torch.Tensor) -> bool:
        return not fsdp_criteria(p) and not hsdp_criteria(p)

    tests = (fsdp_criteria, hsdp_criteria, neither)

    def three_way(items: Iterable[torch.Tensor]):
        items = list(items)
        return tuple([p for p in items if test(p)] for test in tests)

    peek, original = itertools.tee(iter(params))
    first = next(peek)
    if isinstance(first, torch.Tensor):
        return three_way(original)  # type: ignore[return-value]
    if isinstance(first, dict):
        outs: tuple[list, list, list] = ([], [], [])
        for group in original:
            for out, part in zip(outs, three_way(group["params"]), strict=True):  # type: ignore[index]
                out.append({"params": part})
        return outs
    if isinstance(first, tuple):
        named = dict(original)  # type: ignore[arg-type]
        parts = [{k: v for k, v in named.items() if test(v)} for test in tests]
        union = parts[0].keys() | parts[1].keys() | parts[2].keys()
        assert union == named.keys(), f"{union - named.keys()=} {named.keys() - union=}"
        for (na, a), (nb, b) in itertools.combinations(
            zip(("fsdp_params_dict", "hsdp_params_dict", "other_params_dict"), parts), 2
        ):
            assert not (common := a.keys() & b.keys()), f"{common} exist in both {na} and {nb}!"
        return tuple(list(part.items()) for part in parts)  # type: ignore[return-value]
    raise ValueError(
        f"Unsupported params type: {type(first)}. "
        "Please use a list of parameters, parameter groups, or tuples of named parameters."
    )


def parse_fsdp_params(
    params: ParamsT, param_metadata: dict[torch.nn.Parameter, FSDPParameterMetadata]
) -> tuple[ParamsT, ParamsT, ParamsT]:
    """``(FSDP-sharded, HSDP-sharded, other)`` for an FSDP1 model."""

    def strategy_in(p: torch.Tensor, strategies: tuple[ShardingStrategy, ...]) -> bool:
        return isinstance(p, torch.nn.Parameter) and p in param_metadata and param_metadata[p].sharding_strategy in strategies

    return _partition_params(
        params,
        fsdp_criteria=lambda p: strategy_in(p, (ShardingStrategy.FULL_SHARD, ShardingStrategy.SHARD_GRAD_OP)),
        hsdp_criteria=lambda p: strategy_in(p, (ShardingStrategy.HYBRID_SHARD, ShardingStrategy._HYBRID_SHARD_ZERO2)),
    )


def parse_fully_shard_params(params: ParamsT) -> tuple[ParamsT, ParamsT, ParamsT]:
    """``(1-D mesh DTensors, 2-D mesh DTensors, other)`` for a ``fully_shard`` model."""
    return _partition_params(
        params,
        fsdp_criteria=lambda p: isinstance(p, DTensor) and len(p.device_mesh.shape) == 1,
        hsdp_criteria=lambda p: isinstance(p, DTensor) and len(p.device_mesh.shape) == 2,
    )
