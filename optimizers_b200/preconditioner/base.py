"""Interface every preconditioner list implements, plus the profiler-range decorator.

A *preconditioner list* owns the optimizer state of one kind (diagonal second moment, Kronecker
factors, ...) for all blocks a rank works on, and exposes three operations on the sub-list of
blocks that received a gradient this step: update the statistics, apply the preconditioner,
and re-select the active sub-list.

Reference counterpart: ``distributed_shampoo/preconditioner/preconditioner_list.py:23-102``.
"""

from __future__ import annotations

import abc
import functools
from collections.abc import Callable
from typing import Any, TypeVar

import torch
from torch import Tensor
from torch.autograd import profiler

_R = TypeVar("_R")


def profile_decorator(member_func: Callable[..., _R]) -> Callable[..., _R]:
    """Run a method inside a profiler range named ``## Class:method ##``."""

    @functools.wraps(member_func)
    def ranged(self: object, *args: Any, **kwargs: Any) -> _R:
        with profiler.record_function(f"## {type(self).__name__}:{member_func.__name__} ##"):
            return member_func(self, *args, **kwargs)

    return ranged


class PreconditionerList(abc.ABC):
    def __init__(self, block_list: tuple[Tensor, ...]) -> None:
        super().__init__()
        n = len(block_list)
        self._dims_list: tuple[torch.Size, ...] = tuple(b.size() for b in block_list)
        self._numel_list: tuple[int, ...] = (0,) * n
        self._num_bytes_list: tuple[int, ...] = (0,) * n

    @abc.abstractmethod
    def update_preconditioners(
        self, masked_grad_list: tuple[Tensor, ...], step: Tensor, perform_amortized_computation: bool
    ) -> None: ...

    @abc.abstractmethod
    def precondition(self, masked_grad_list: tuple[Tensor, ...]) -> tuple[Tensor, ...]: ...

    @abc.abstractmethod
    def compress_preconditioner_list(self, local_grad_selector: tuple[bool, ...]) -> None: ...

    @property
    def numel_list(self) -> tuple[int, ...]:
        return self._numel_list

    @property
    def dims_list(self) -> tuple[torch.Size, ...]:
        return self._dims_list

    @property
    def num_bytes_list(self) -> tuple[int, ...]:
        return self._num_bytes_list

    def numel(self) -> int:
        return sum(self._numel_list)

    def num_bytes(self) -> int:
        return sum(self._num_bytes_list)
