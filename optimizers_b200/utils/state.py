"""Checkpointable optimizer-state containers and the helpers that move them in and out of
``optimizer.state_dict()``.

``OptimizerModule`` plays the role ``nn.Module`` plays for models: an object whose attributes
(tensors, nested modules, dicts, sequences) serialise into a nested dict of tensors and load back
*in place*, so views and aliases held elsewhere (kernel block tables, arenas) stay valid.
Sequences become ``{index: value}`` dicts; after a round trip through flattened distributed
checkpoints the integer keys come back as strings and are repaired on load.

Reference counterparts: ``distributed_shampoo/utils/optimizer_modules.py:23-248`` and
``distributed_shampoo/utils/shampoo_state_dict_utils.py:21-73``.
"""

from __future__ import annotations

import logging
from copy import deepcopy
from typing import Any

import torch
from torch import Tensor

logger: logging.Logger = logging.getLogger(__name__)

_CONTAINERS = (list, tuple, set)


def _emit(value: Any, keep_vars: bool, store_non_tensors: bool) -> tuple[bool, Any]:
    """Serialise one attribute.  Returns ``(present, payload)``; containers that serialise to
    nothing are dropped, non-tensor leaves are dropped unless asked for."""
    if isinstance(value, Tensor):
        return True, (value if keep_vars else value.detach())
    if isinstance(value, OptimizerModule):
        return True, value.state_dict(keep_vars=keep_vars, store_non_tensors=store_non_tensors)
    if isinstance(value, dict) or isinstance(value, _CONTAINERS):
        items = value.items() if isinstance(value, dict) else enumerate(value)
        out = {}
        for k, v in items:
            present, payload = _emit(v, keep_vars, store_non_tensors)
            if present:
                out[k] = payload
        return bool(out), out
    return store_non_tensors, value


def _int_keys(template_len: int, incoming: dict) -> dict[int, Any]:
    """Sequence payloads are keyed by position; accept ``"0"``-style keys as well."""
    if incoming and all(isinstance(k, int) for k in incoming):
        return incoming
    fixed = {}
    for i in range(template_len):
        if str(i) not in incoming:
            raise KeyError(f"Index {i} not found in new_state. new_state keys: {incoming.keys()}")
        fixed[i] = incoming[str(i)]
    return fixed


def _absorb(current: Any, incoming: Any, store_non_tensors: bool) -> Any:
    """Load ``incoming`` into ``current`` and return the object that should now be stored."""
    if isinstance(current, Tensor):
        if not isinstance(incoming, Tensor):
            logger.warning(
                f"Both old state {current} and new state {incoming} must be tensors! Continuing..."
            )
            return current
        current.detach().copy_(incoming)
        return current
    if isinstance(current, OptimizerModule):
        current.load_state_dict(incoming, store_non_tensors)
        return current
    if isinstance(current, dict):
        if not isinstance(incoming, dict):
            logger.warning(
                f"Both old state {current} and new_state {incoming} must be dicts! Continuing..."
            )
            return current
        for key in list(current.keys()):
            if key in incoming:
                current[key] = _absorb(current[key], incoming[key], store_non_tensors)
        return current
    if isinstance(current, _CONTAINERS):
        if isinstance(incoming, dict) and incoming:
            incoming = _int_keys(len(current), incoming)
        rebuilt = []
        for i, item in enumerate(current):
            structured = isinstance(item, (Tensor, dict, OptimizerModule) + _CONTAINERS)
            if structured or store_non_tensors:
                rebuilt.append(_absorb(item, incoming[i], store_non_tensors))
            else:
                rebuilt.append(item)
        return type(current)(rebuilt)
    if store_non_tensors:
        if type(current) is not type(incoming):
            logger.warning(
                f"Types of old value {type(current)} and new value {type(incoming)} do not match! Continuing..."
            )
            return current
        return deepcopy(incoming)
    return current


class OptimizerModule:
    """Base class for checkpointable optimizer state; see the module docstring."""

    def state_dict(
        self,
        destination: dict | None = None,
        keep_vars: bool = False,
        store_non_tensors: bool = False,
    ) -> dict:
        if destination is None:
            destination = {}
        for key, value in self.__dict__.items():
            if isinstance(value, (Tensor, OptimizerModule)):
                destination[key] = _emit(value, keep_vars, store_non_tensors)[1]
                continue
            present, payload = _emit(value, keep_vars, store_non_tensors)
            if present:
                destination[key] = payload
        return destination

    def load_state_dict(self, state_dict: dict, store_non_tensors: bool = False) -> None:
        _absorb(self.__dict__, state_dict, store_non_tensors)


def update_param_state_dict_object(
    current_param_state_dict: dict[str, Any],
    param_state_dict_to_load: dict[str, Any],
    enable_missing_key_check: bool = True,
) -> None:
    """Copy a loaded per-parameter state tree into the live one without replacing its tensors or
    modules."""
    for key, live in current_param_state_dict.items():
        if key not in param_state_dict_to_load:
            if enable_missing_key_check:
                raise KeyError(f"Key {key} not found in state dict to load.")
            logger.warning(f"Key {key} not found in state dict to load.")
            continue
        loaded = param_state_dict_to_load[key]
        if isinstance(live, dict):
            update_param_state_dict_object(live, loaded, enable_missing_key_check)
        elif callable(getattr(live, "load_state_dict", None)):
            live.load_state_dict(loaded)
        elif isinstance(live, Tensor):
            live.detach().copy_(loaded)
        else:
            current_param_state_dict[key] = deepcopy(loaded)


def extract_state_dict_content(input_dict: dict[str, Any]) -> dict[str, Any]:
    """Replace every ``OptimizerModule`` inside a state tree by its ``state_dict()``."""

    def convert(value: Any) -> Any:
        if isinstance(value, dict):
            return extract_state_dict_content(value)
        if isinstance(value, OptimizerModule):
            return value.state_dict()
        return value

    return {k: convert(v) for k, v in input_dict.items()}
