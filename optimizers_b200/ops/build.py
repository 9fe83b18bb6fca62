"""In-tree build and loading of the sm_100a CUDA extension.

``build()`` compiles ``csrc/*.cu`` with nvcc for ``compute_100a/sm_100a`` into
``optimizers_b200/ops/_C.so`` (cross-compilation works without a GPU).  ``load()`` imports the
built module; it never compiles implicitly on a machine that has a GPU but no toolchain cache,
and it raises when the module is missing so that GPU code paths cannot fall back silently.
"""

from __future__ import annotations

import importlib.util
import os
import shutil
import sys
from pathlib import Path
from types import ModuleType

_HERE = Path(__file__).resolve().parent
_CSRC = _HERE / "csrc"
_NAME = "optimizers_b200_C"
_SO = _HERE / f"{_NAME}.so"
_module: ModuleType | None = None

SOURCES = ["bindings.cu", "grouped_gemm.cu", "block_kernels.cu", "flat_kernels.cu", "eig_kernels.cu", "two_sided_apply.cu", "model_kernels.cu"]
NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-Xptxas=-v",
    "-std=c++17",
]


def _stale() -> bool:
    if not _SO.exists():
        return True
    built = _SO.stat().st_mtime
    return any(p.stat().st_mtime > built for p in _CSRC.iterdir() if p.suffix in (".cu", ".cuh", ".h"))


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the extension if it is missing or older than its sources; return the .so path."""
    if not force and not _stale():
        return _SO
    from torch.utils import cpp_extension

    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    build_dir = _HERE / "build"
    build_dir.mkdir(exist_ok=True)
    cpp_extension.load(
        name=_NAME,
        sources=[str(_CSRC / s) for s in SOURCES],
        extra_include_paths=[str(_CSRC)],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        build_directory=str(build_dir),
        verbose=verbose,
        is_python_module=False,
    )
    shutil.copyfile(build_dir / f"{_NAME}.so", _SO)
    return _SO


def available() -> bool:
    return _SO.exists()


def load() -> ModuleType:
    """Import the built extension (building it first only when a compiler is at hand and the
    module is missing)."""
    global _module
    if _module is not None:
        return _module
    if not _SO.exists():
        if shutil.which("nvcc") is None:
            raise RuntimeError(
                f"The sm_100a extension {_SO} has not been built and no nvcc is available; "
                "run `make build` where the CUDA toolkit is installed."
            )
        build()
    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location(_NAME, _SO)
    assert spec is not None and spec.loader is not None
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[_NAME] = module
    _module = module
    from optimizers_b200.utils import tracing

    tracing.configure_from_environment()
    return module
