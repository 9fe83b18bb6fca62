"""Tracing of the native launches.

The reference marks its phases with ``torch.profiler.record_function`` only
(distributed_shampoo/preconditioner/preconditioner_list.py:23-55); its work is ATen kernels, which
profilers name by themselves.  Here the work is this package's own kernels, so the bindings can
wrap every launch in an NVTX range (``ob200::grouped_gemm``, ``ob200::grad_prologue``, ...) and can
bracket it with CUDA events that accumulate device time per binding:

    from optimizers_b200.utils import tracing
    tracing.enable(nvtx=True, timing=True)
    ... training steps ...
    for name, (calls, ms) in tracing.launch_timings(reset=True).items(): ...

``OB200_TRACE=nvtx``, ``=timing`` or ``=nvtx,timing`` in the environment enables the same when the
extension is loaded.  The native engine additionally emits an NVTX marker at each phase boundary of
its step while NVTX tracing is on.
"""

from __future__ import annotations

import os

_nvtx = False
_timing = False


def _apply() -> None:
    from optimizers_b200.ops import build

    if build.available():
        build.load().set_launch_tracing(_nvtx, _timing)


def enable(nvtx: bool = True, timing: bool = False) -> None:
    global _nvtx, _timing
    _nvtx, _timing = bool(nvtx), bool(timing)
    _apply()


def disable() -> None:
    enable(False, False)


def nvtx_enabled() -> bool:
    return _nvtx


def launch_timings(reset: bool = False) -> dict[str, tuple[int, float]]:
    """``{binding name: (calls, device milliseconds)}`` accumulated while timing was enabled.
    Waits for the recorded events, so call it outside the timed region."""
    from optimizers_b200.ops import build

    if not build.available():
        return {}
    return {k: (int(c), float(ms)) for k, (c, ms) in build.load().launch_timings(reset).items()}


def configure_from_environment() -> None:
    spec = {s.strip() for s in os.environ.get("OB200_TRACE", "").split(",") if s.strip()}
    if spec:
        enable(nvtx="nvtx" in spec, timing="timing" in spec)
