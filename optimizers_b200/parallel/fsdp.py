"""FSDP1 (flat-parameter ``FULL_SHARD``) distributor.

Under FSDP1 each rank holds a contiguous 1-D slice ``[start_idx, end_idx)`` of every flattened
original parameter.  A slice generally is not a rectangle of the original tensor, so it is cut
into the largest rectangular pieces it contains (``recover_rectangles``) and every piece is
blocked and preconditioned on its own, locally, without optimizer communication.  The result
differs numerically from unsharded Shampoo because the blocks differ.

Reference counterpart: ``distributed_shampoo/distributor/shampoo_fsdp_distributor.py:36-405``.
"""

from __future__ import annotations

import math
from typing import Any

import torch
from torch import distributed as dist, Tensor
from torch.nn.parameter import Parameter

from optimizers_b200.config import DISTRIBUTED_CONFIG, FSDPDistributedConfig, FSDPParameterMetadata, PARAMS, ShampooRuntimeConfig
from optimizers_b200.parallel.base import Distributor
from optimizers_b200.parallel.block_info import BlockInfo
from optimizers_b200.utils.blocking import compress_list, generate_pairwise_indices


def recover_rectangles(shape: tuple[int, ...], start: int, end: int) -> list[tuple[int, tuple[int, ...]]]:
    """Cut the flat index range ``[start, end)`` of a row-major tensor of ``shape`` into maximal
    rectangular pieces.  Returns ``(flat start index, piece shape)`` in ascending order.

    At depth ``dim`` a "row" spans ``r = prod(shape[dim+1:])`` elements.  Whole rows inside the
    range form one piece of shape ``(rows, *shape[dim+1:])``; the ragged ends before and after
    are handled one depth further down; a range without a row boundary goes down as a whole."""

    def rec(dim: int, lo: int, hi: int) -> list[tuple[int, tuple[int, ...]]]:
        if lo == hi:
            return []
        if dim == len(shape) - 1:
            return [(lo, (hi - lo,))]
        r = math.prod(shape[dim + 1 :])
        first = -(-lo // r) * r  # first row boundary at or after lo
        last = hi // r * r  # last row boundary at or before hi
        if first > last:
            return rec(dim + 1, lo, hi)
        centre = [(first, ((last - first) // r, *shape[dim + 1 :]))] if first < last else []
        return rec(dim + 1, lo, first) + centre + rec(dim + 1, last, hi)

    return rec(0, start, end)


class FlatShardBlocking:
    """Blocking of FSDP1 flat-parameter shards, shared by the FSDP and HSDP distributors.
    Expects ``self._param_to_metadata`` and the ``DistributorInterface`` helpers."""

    _param_to_metadata: dict[Parameter, FSDPParameterMetadata]

    @staticmethod
    def _split_tensor_block_recovery(
        tensor_shard: Tensor, original_shape: torch.Size, start_idx: int, end_idx: int
    ) -> list[Tensor]:
        if tensor_shard.dim() != 1:
            raise ValueError(f"Input tensor is not flat, has shape tensor_shard.size()={tensor_shard.size()}.")
        assert end_idx - start_idx == tensor_shard.numel(), (
            f"Start/end indices do not match tensor size: block_start_idx={start_idx}, "
            f"block_end_idx={end_idx}, block_within_tensor_shard.numel()={tensor_shard.numel()}!"
        )
        return [
            tensor_shard.narrow(0, flat_start - start_idx, math.prod(piece_shape)).view(piece_shape)
            for flat_start, piece_shape in recover_rectangles(tuple(original_shape), start_idx, end_idx)
        ]

    def _pieces_of(self, flat_param: Tensor, tensor: Tensor) -> list[Tensor]:
        meta = self._param_to_metadata[flat_param]  # type: ignore[index]
        return self._split_tensor_block_recovery(tensor, meta.shape, meta.start_idx, meta.end_idx)

    def _merge_and_block_parameters(self) -> None:
        blocks: list[Tensor] = []
        splits_per_param: list[int] = []
        blocks_per_split: list[int] = []
        for flat in self._param_group[PARAMS]:  # type: ignore[attr-defined]
            pieces = self._pieces_of(flat, flat)
            splits_per_param.append(len(pieces))
            piece_blocks, counts = self._merge_and_block_with_params(pieces)  # type: ignore[attr-defined]
            blocks.extend(piece_blocks)
            blocks_per_split.extend(counts)
        self._global_blocked_params = tuple(blocks)
        self._global_num_splits_per_param = tuple(splits_per_param)
        self._global_num_blocks_per_split_param = tuple(blocks_per_split)
        self._global_num_blocks_per_param = tuple(
            sum(blocks_per_split[lo:hi]) for lo, hi in generate_pairwise_indices(splits_per_param)
        )

    def _merge_and_block_gradients(self) -> tuple[Tensor, ...]:
        local_grads: list[Tensor] = []
        selector: list[bool] = []
        for flat, count, (blo, bhi), (slo, shi) in zip(
            self._param_group[PARAMS],  # type: ignore[attr-defined]
            self._global_num_blocks_per_param,
            generate_pairwise_indices(self._global_num_blocks_per_param),
            generate_pairwise_indices(self._global_num_splits_per_param),
            strict=True,
        ):
            grad = flat.grad
            mine = self._distributor_selector[blo:bhi]  # type: ignore[attr-defined]
            usable = grad is not None and grad.numel() > 0
            selector.extend([usable] * count)
            if not usable or not any(mine):
                continue
            if self._runtime_config.eager_nan_check:  # type: ignore[attr-defined]
                assert torch.isfinite(grad).all(), (
                    f"Encountered gradient containing NaN/Inf in parameter with shape {grad.shape}. Check your model for numerical instability or consider gradient clipping."
                )
            per_piece_counts = self._global_num_blocks_per_split_param[slo:shi]
            for piece, (lo, hi) in zip(
                self._pieces_of(flat, grad), generate_pairwise_indices(per_piece_counts), strict=True
            ):
                local_grads.extend(compress_list(self._blocks_of(piece), mine[lo:hi]))  # type: ignore[attr-defined]
        self._global_grad_selector = tuple(selector)
        return tuple(local_grads)


class FSDPDistributor(FlatShardBlocking, Distributor):
    def __init__(self, param_group: dict[str, Any], runtime_config: ShampooRuntimeConfig | None = None) -> None:
        cfg: FSDPDistributedConfig = param_group[DISTRIBUTED_CONFIG]
        self._param_to_metadata = cfg.param_to_metadata
        self._global_num_splits_per_param: tuple[int, ...] = ()
        self._global_num_blocks_per_split_param: tuple[int, ...] = ()
        super().__init__(param_group, runtime_config)

    @torch.no_grad()
    def _construct_local_block_info_list(self) -> tuple[BlockInfo, ...]:
        # Block ids carry the rank: the same parameter has different blocks on different ranks.
        return self._construct_local_block_info_list_with_params(
            params=self._get_params_or_grads(), rank=dist.get_rank()
        )
