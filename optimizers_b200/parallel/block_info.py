"""Per-block metadata handed from a distributor to the preconditioners.

A block is a view into a parameter (or into a local shard of it).  ``BlockInfo`` records which
parameter the block came from, its ``(param_index, block_id)`` pair -- the block id is the key
under ``optimizer.state[param]`` -- and four callables that let state be allocated either as
plain tensors or as ``DTensor`` replicated over the owner's sub-mesh:

* ``allocate_zeros_tensor(size, dtype, device)``
* ``allocate_ones_tensor(size, dtype, device)``
* ``allocate_eye_tensor(n, dtype, device)``
* ``get_tensor(t)`` -- the local plain tensor behind ``t``.

Reference counterpart: ``distributed_shampoo/distributor/shampoo_block_info.py:18-135``.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass, field

import torch
from torch import Tensor


def _identity(t: Tensor) -> Tensor:
    return t


def _to_local(t: Tensor) -> Tensor:
    return t.to_local()  # type: ignore[attr-defined]


@dataclass
class BlockInfo:
    param: Tensor
    composable_block_ids: tuple[int, str]
    allocate_zeros_tensor: Callable[..., Tensor] = torch.zeros
    allocate_ones_tensor: Callable[..., Tensor] = field(init=False, default_factory=lambda: torch.ones)
    allocate_eye_tensor: Callable[..., Tensor] = field(init=False, default_factory=lambda: torch.eye)
    get_tensor: Callable[..., Tensor] = field(init=False, default_factory=lambda: _identity)


@dataclass
class DTensorBlockInfo(BlockInfo):
    """State is allocated through ``allocate_zeros_tensor`` (a DTensor factory supplied by the
    distributor); ones and identity are derived from it by filling the local tensor."""

    get_tensor: Callable[..., Tensor] = field(init=False, default_factory=lambda: _to_local)

    def __post_init__(self) -> None:
        def ones(size, dtype=None, device=None) -> Tensor:
            t = self.allocate_zeros_tensor(size=size, dtype=dtype, device=device)
            self.get_tensor(t).fill_(1.0)
            return t

        def eye(n, dtype=None, device=None) -> Tensor:
            t = self.allocate_zeros_tensor(size=(n, n), dtype=dtype, device=device)
            self.get_tensor(t).fill_diagonal_(1.0)
            return t

        self.allocate_ones_tensor = ones
        self.allocate_eye_tensor = eye
