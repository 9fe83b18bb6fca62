"""Small helper idioms: subclass discovery, batching, lock-step iteration over a dict of
iterables.

Reference counterparts: ``distributed_shampoo/utils/commons.py:20-76`` and
``distributed_shampoo/utils/dict_zip_iterator.py:16-109``.
"""

from __future__ import annotations

from collections.abc import Iterable, Iterator
from itertools import islice
from typing import Generic, TypeVar

_T = TypeVar("_T")


def get_all_non_abstract_subclasses(cls: type) -> Iterable[type]:
    """Every concrete class at or below ``cls`` in the inheritance graph (each once)."""
    seen: set[type] = set()
    stack = [cls]
    while stack:
        c = stack.pop()
        if c in seen:
            continue
        seen.add(c)
        stack.extend(c.__subclasses__())
    return (c for c in seen if not getattr(c, "__abstractmethods__", frozenset()))


def batched(iterable: Iterable[_T], n: int) -> Iterable[tuple[_T, ...]]:
    """Consecutive tuples of up to ``n`` items."""
    if n < 1:
        raise ValueError(f"n={n} must be at least one")
    it = iter(iterable)
    while chunk := tuple(islice(it, n)):
        yield chunk


class DictZipIterator(Generic[_T], Iterator[dict[str, _T]]):
    """``zip`` over the values of a dict, yielding dicts; all iterables must have equal length."""

    def __init__(self, data: dict[str, Iterable[_T]]) -> None:
        self._iterators = {k: iter(v) for k, v in data.items()}

    def __iter__(self) -> "DictZipIterator[_T]":
        return self

    def __next__(self) -> dict[str, _T]:
        row: dict[str, _T] = {}
        finished = []
        for key, it in self._iterators.items():
            try:
                row[key] = next(it)
            except StopIteration:
                finished.append(key)
        if finished and row:
            raise ValueError(f"Iterators have different lengths. Exhausted: {finished}, Still active: {list(row)}")
        if finished:
            raise StopIteration
        return row
