"""Shape merging, blocking, selection, symmetric packing and load-balancing primitives.

These are the host-side index computations every distributor and preconditioner shares.
Behaviour parity (tie-breaking included, because it decides block ownership and therefore the
checkpoint layout) with the reference's ``distributed_shampoo/utils/shampoo_utils.py``:
``merge_small_dims`` (:38-121), ``multi_dim_split`` (:124-174), ``compress_list`` (:180-205),
``distribute_buffer_sizes`` (:282-344), ``pack/unpack_upper_triangular`` (:1178-1249),
``greedy_bin_pack`` (:1255-1289), ``split_param_groups`` (:1292-1591).
"""

from __future__ import annotations

import copy
import heapq
import itertools
import logging
import math
from collections.abc import Callable, Iterator, Sequence
from functools import cache
from types import TracebackType
from typing import Any, TypeVar

import torch
from torch import Tensor

from optimizers_b200.config import (
    DefaultCostModel,
    DISTRIBUTED_CONFIG,
    FSDPParamAssignmentStrategy,
    FullyShardDistributedConfig,
    HybridShardDistributedConfig,
    LoadBalancingConfig,
    OWNER_RANKS,
    PARAMS,
)

logger: logging.Logger = logging.getLogger(__name__)

_T = TypeVar("_T")


# --------------------------------------------------------------------------------------------
# Shapes and blocks
# --------------------------------------------------------------------------------------------
@cache
def merge_small_dims(
    tensor_shape: tuple[int, ...],
    threshold: int | float,
    target_tensor_dimensionality: int | float = 1,
) -> tuple[int, ...]:
    """Collapse neighbouring dims (scanning from the last dim towards the first) while the merged
    extent stays ≤ ``threshold`` and the tensor would otherwise have more than
    ``target_tensor_dimensionality`` dims.  Size-1 dims vanish; any 0 extent gives ``(0,)``;
    a scalar gives ``(1,)``; ``math.inf`` as target returns the shape untouched."""
    if 0 in tensor_shape:
        return (0,)
    if isinstance(target_tensor_dimensionality, float):
        assert target_tensor_dimensionality == math.inf, (
            f"{target_tensor_dimensionality=} has to be an integer or math.inf."
        )
        return tensor_shape

    # Work on the reversed, squeezed shape so that merging proceeds right-to-left.
    dims = [d for d in reversed(tensor_shape) if d != 1] or [1]
    merged = [dims[0]]
    for seen, extent in enumerate(dims[1:], start=1):
        dims_if_no_merge = len(merged) + (len(dims) - seen)
        candidate = merged[-1] * extent
        if dims_if_no_merge > target_tensor_dimensionality and candidate <= threshold:
            merged[-1] = candidate
        else:
            merged.append(extent)
    merged.reverse()
    return tuple(merged)


def multi_dim_split(tensor: Tensor, split_size: int | float) -> tuple[Tensor, ...]:
    """Chop ``tensor`` into blocks of at most ``split_size`` along every dim; blocks are views
    and come out in row-major block order."""
    if isinstance(split_size, float):
        assert split_size == math.inf, f"{split_size=} has to be an integer or math.inf."
        return (tensor,)
    pieces: tuple[Tensor, ...] = (tensor,)
    for dim in range(tensor.dim()):
        pieces = tuple(s for t in pieces for s in torch.split(t, split_size, dim=dim))
    return pieces


def block_slices(
    shape: tuple[int, ...], split_size: int | float
) -> list[tuple[tuple[int, int], ...]]:
    """Index-only twin of :func:`multi_dim_split`: for every block, its ``(start, stop)`` per dim,
    in the same order.  Used to build device block tables without touching tensors."""
    if isinstance(split_size, float):
        return [tuple((0, d) for d in shape)]
    per_dim = [
        [(s, min(s + split_size, d)) for s in range(0, d, split_size)] or [(0, 0)] for d in shape
    ]
    return [tuple(combo) for combo in itertools.product(*per_dim)]


def compress_list(complete_list: Sequence[_T], selector: Sequence[bool]) -> tuple[_T, ...]:
    """Keep the entries whose selector bit is set."""
    assert len(complete_list) == len(selector), (
        f"Inconsistent lengths between complete_list {len(complete_list)} and selector {len(selector)}!"
    )
    return tuple(itertools.compress(complete_list, selector))


def get_dtype_size(dtype: torch.dtype) -> int:
    """Bytes per element."""
    if dtype is torch.bool:
        return 1
    info = torch.finfo(dtype) if dtype.is_floating_point else torch.iinfo(dtype)
    return (info.bits + 7) // 8


def generate_pairwise_indices(input_list: Sequence[int]) -> Iterator[tuple[int, int]]:
    """``[a, b, c]`` → ``(0, a), (a, a+b), (a+b, a+b+c)``: the index range of each run."""
    return itertools.pairwise(itertools.accumulate(itertools.chain([0], input_list)))


class ParameterizeEnterExitContext:
    """Context manager built from two callables applied to one object on enter and on exit
    (for example ``optimizer.eval()`` around a checkpoint save, ``optimizer.train()`` after)."""

    def __init__(
        self,
        input_with_enter_exit_context: _T,
        enter_method_caller: Callable[[_T], Any],
        exit_method_caller: Callable[[_T], Any],
    ) -> None:
        self._obj = input_with_enter_exit_context
        self._on_enter = enter_method_caller
        self._on_exit = exit_method_caller

    def __enter__(self) -> "ParameterizeEnterExitContext":
        self._on_enter(self._obj)
        return self

    def __exit__(
        self,
        exc_type: type[BaseException] | None,
        exc_val: BaseException | None,
        exc_tb: TracebackType | None,
    ) -> None:
        self._on_exit(self._obj)


# --------------------------------------------------------------------------------------------
# Load balancing (longest-processing-time-first onto the least loaded rank)
# --------------------------------------------------------------------------------------------
def lpt_assign(costs: Sequence[float], num_bins: int, initial_loads: Sequence[float] | None = None):
    """Greedy LPT.  Items are visited by descending cost (stable: equal costs keep their original
    order) and each goes to the bin with the smallest ``(load, bin index)``.  Returns
    ``(owner per item, final load per bin)``."""
    heap = [(float(initial_loads[b]) if initial_loads is not None else 0.0, b) for b in range(num_bins)]
    heapq.heapify(heap)
    owners = [-1] * len(costs)
    for index in sorted(range(len(costs)), key=lambda i: costs[i], reverse=True):
        load, b = heapq.heappop(heap)
        owners[index] = b
        heapq.heappush(heap, (load + costs[index], b))
    loads = [0.0] * num_bins
    for load, b in heap:
        loads[b] = load
    return owners, loads


def distribute_buffer_sizes(
    blocked_params: tuple[Tensor, ...],
    group_size: int,
    load_balancing_config: LoadBalancingConfig,
) -> tuple[tuple[int, int], ...]:
    """For every block: ``(64-byte aligned byte size, owner rank in the group)``.  The size is
    always the aligned memory footprint; the owner is chosen by LPT on the configured cost."""
    sizes = [int(DefaultCostModel.cost(b)) for b in blocked_params]
    costs = [load_balancing_config.cost_model.cost(b) for b in blocked_params]
    owners, _ = lpt_assign(costs, group_size)
    return tuple(zip(sizes, owners, strict=True))


def greedy_bin_pack(
    items: Sequence[_T], num_bins: int, cost_fn: Callable[[_T], int]
) -> tuple[list[list[_T]], list[int]]:
    """LPT bin packing that returns the bins themselves.  Among equal costs the *later* item is
    placed first (the sort key is ``(cost, position)`` descending)."""
    bins: list[list[_T]] = [[] for _ in range(num_bins)]
    heap = [(0, b) for b in range(num_bins)]
    heapq.heapify(heap)
    keyed = sorted(((cost_fn(it), pos) for pos, it in enumerate(items)), reverse=True)
    for cost, pos in keyed:
        load, b = heapq.heappop(heap)
        bins[b].append(items[pos])
        heapq.heappush(heap, (load + cost, b))
    bin_costs = [0] * num_bins
    for load, b in heap:
        bin_costs[b] = load
    return bins, bin_costs


# --------------------------------------------------------------------------------------------
# Symmetric packing: row-major upper triangle, d(d+1)/2 entries
# --------------------------------------------------------------------------------------------
def _device_key(device: torch.device) -> tuple[str, int]:
    if device.type == "cuda" and device.index is None:
        return ("cuda", torch.cuda.current_device())
    return (device.type, device.index or 0)


@cache
def _triu_index_pair(d: int, device_type: str, device_index: int) -> Tensor:
    # int32 halves the index traffic; cached because rebuilding it every step is measurable.
    dev = torch.device(device_type, device_index)
    return torch.triu_indices(d, d, device=dev).to(torch.int32)


def packed_size(d: int) -> int:
    return d * (d + 1) // 2


def packed_row_offset(i: int, d: int) -> int:
    """Offset of element (i, i) in the packed row-major upper triangle of a d×d matrix."""
    return i * d - i * (i - 1) // 2


def pack_upper_triangular(matrix: Tensor) -> Tensor:
    rows, cols = _triu_index_pair(matrix.shape[0], *_device_key(matrix.device))
    return matrix[rows, cols].contiguous()


def unpack_upper_triangular(packed: Tensor, dim: int) -> Tensor:
    full = torch.zeros(dim, dim, dtype=packed.dtype, device=packed.device)
    rows, cols = _triu_index_pair(dim, *_device_key(packed.device))
    full[rows, cols] = packed
    full[cols, rows] = packed
    return full


# --------------------------------------------------------------------------------------------
# Param-group splitting for the lossless FSDP/HSDP distributors
# --------------------------------------------------------------------------------------------
def _shard_group_size(cfg: FullyShardDistributedConfig) -> int:
    if isinstance(cfg, HybridShardDistributedConfig):
        return cfg.device_mesh.size(1)
    return torch.distributed.get_world_size()


def _compute_global_owner_ranks(
    params: Sequence[Tensor], distributed_config: FullyShardDistributedConfig
) -> list[int]:
    """Owner rank (within the shard group) of each whole parameter under ROUND_ROBIN."""
    pairs = distribute_buffer_sizes(
        tuple(params), _shard_group_size(distributed_config), distributed_config.load_balancing_config
    )
    return [rank for _, rank in pairs]


def _compute_per_bucket_owner_ranks(
    buckets: list[list[int]], params: Sequence[Tensor], distributed_config: FullyShardDistributedConfig
) -> list[list[int]]:
    """LPT inside each bucket, with the per-rank load carried from bucket to bucket so that the
    total stays balanced although each bucket is balanced on its own."""
    n = _shard_group_size(distributed_config)
    cost_model = distributed_config.load_balancing_config.cost_model
    loads = [0.0] * n
    result = []
    for bucket in buckets:
        costs = [float(cost_model.cost(params[i])) for i in bucket]
        owners, loads = lpt_assign(costs, n, initial_loads=loads)
        result.append(owners)
    return result


def _create_sub_groups(group: dict[str, Any], n: int, is_round_robin: bool = False) -> list[dict[str, Any]]:
    params = group[PARAMS]
    cfg = group[DISTRIBUTED_CONFIG]
    buckets, _ = greedy_bin_pack(list(range(len(params))), n, cost_fn=lambda i: params[i].numel())
    if isinstance(cfg, HybridShardDistributedConfig):
        shard_size = cfg.device_mesh.size(1)
        for i, bucket in enumerate(buckets):
            if bucket and len(bucket) < shard_size:
                raise ValueError(
                    f"HSDP sub-group {i} got {len(bucket)} params after "
                    f"greedy bin-packing, fewer than shard_size={shard_size}. "
                    "This happens when one or more params dominate by numel, "
                    "leaving a degenerate tiny sub-group. This is an efficiency "
                    "guard, not a correctness/deadlock requirement -- shard ranks "
                    "owning zero params still participate via all_to_all padding. "
                    "Reduce num_sub_groups or rebalance the param shapes."
                )
    owners = _compute_per_bucket_owner_ranks(buckets, params, cfg) if is_round_robin else None
    shared = {k: v for k, v in group.items() if k not in (PARAMS, OWNER_RANKS)}
    out = []
    for b, bucket in enumerate(buckets):
        if not bucket:
            continue
        sub = {**shared, PARAMS: [params[i] for i in bucket], DISTRIBUTED_CONFIG: copy.copy(cfg)}
        if owners is not None:
            sub[OWNER_RANKS] = owners[b]
        out.append(sub)
    return out


def split_param_groups(param_groups: list[dict[str, Any]]) -> list[dict[str, Any]]:
    """Expand every lossless FSDP/HSDP group with ``num_sub_groups > 1`` into that many groups
    (balanced by numel) so each gets its own distributor, communicator and stream; attach
    ``owner_ranks`` to ROUND_ROBIN groups.  Other groups pass through unchanged."""
    result: list[dict[str, Any]] = []
    for group in param_groups:
        cfg = group[DISTRIBUTED_CONFIG]
        is_fs = isinstance(cfg, FullyShardDistributedConfig)
        round_robin = is_fs and cfg.param_assignment_strategy == FSDPParamAssignmentStrategy.ROUND_ROBIN
        if not (is_fs and cfg.num_sub_groups > 1):
            if round_robin:
                result.append({**group, OWNER_RANKS: _compute_global_owner_ranks(group[PARAMS], cfg)})
            else:
                result.append(group)
            continue
        n = cfg.num_sub_groups
        num_params = len(group[PARAMS])
        shard_size = cfg.device_mesh.size(1) if isinstance(cfg, HybridShardDistributedConfig) else 1
        max_groups = max(1, num_params // shard_size)
        if n > max_groups:
            raise ValueError(
                f"num_sub_groups={n} is too large for {num_params} params with "
                f"shard_group_size={shard_size}: each sub-group should hold at least "
                f"{shard_size} params to avoid degenerate tiny sub-groups (an "
                "efficiency guard, not a correctness/deadlock requirement -- "
                "zero-owner shard ranks are handled by all_to_all padding). "
                f"Maximum num_sub_groups={max_groups}."
            )
        subs = _create_sub_groups(group, n, is_round_robin=round_robin)
        result.extend(subs)
        logger.info(
            "Split param group (%d params) into %d sub-groups (numel per group: %s).",
            num_params,
            len(subs),
            [sum(p.numel() for p in g[PARAMS]) for g in subs],
        )
    return result
