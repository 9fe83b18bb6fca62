"""Selection of the native sm_100a execution engine for a parameter group (stub filled in by
``optimizers_b200.native_engine`` when the CUDA extension is available)."""

from __future__ import annotations

from typing import Any

from optimizers_b200.config import NativeRuntimeConfig, PARAMS


def maybe_build_native_engine(optimizer: Any, rec: dict[str, Any], group: dict[str, Any], cfg: NativeRuntimeConfig):
    """Return a native engine for the group, or ``None`` to use the torch step.

    ``backend="torch"`` and non-CUDA groups always get ``None``.  ``backend="native"`` raises when
    the group cannot be covered; ``"auto"`` falls back silently."""
    if cfg.backend == "torch" or group[PARAMS][0].device.type != "cuda":
        if cfg.backend == "native":
            raise RuntimeError("native backend requested for a parameter group that is not on a CUDA device")
        return None
    from optimizers_b200.native_engine import build_native_engine

    return build_native_engine(optimizer, rec, group, cfg)
