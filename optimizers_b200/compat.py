"""Loading checkpoints written by the reference library.

``optimizer.state_dict()`` of the reference pickles its configuration dataclasses into
``param_groups`` under the module paths ``distributed_shampoo.shampoo_types`` and
``distributed_shampoo.preconditioner.matrix_functions_types``.  A process that only has this
framework installed cannot unpickle such a file.  ``install_reference_aliases()`` registers
stand-in modules under those paths whose attributes are this framework's classes of the same
names (all of them live in ``optimizers_b200.config`` and have the same fields), after which
``torch.load(path, weights_only=False)`` yields a state dict that
``DistributedShampoo.load_state_dict`` accepts unchanged: the state layout (block ids, tensor
names, packing) is the reference's (``distributed_shampoo/distributed_shampoo.py:1850-1996``).

Nothing is registered when the real ``distributed_shampoo`` package is importable or already
imported: the aliases are for processes without it.
"""

from __future__ import annotations

import importlib.util
import sys
import types

_ALIASED = (
    "distributed_shampoo",
    "distributed_shampoo.shampoo_types",
    "distributed_shampoo.preconditioner",
    "distributed_shampoo.preconditioner.matrix_functions_types",
)


def install_reference_aliases(force: bool = False) -> bool:
    """Make the reference's pickled class paths resolve to this framework's classes.  Returns
    True when the aliases are (now) in place, False when the real package is present and
    ``force`` is not set."""
    if "distributed_shampoo" in sys.modules and not getattr(sys.modules["distributed_shampoo"], "__ob200_alias__", False):
        return False
    if not force and "distributed_shampoo" not in sys.modules and importlib.util.find_spec("distributed_shampoo") is not None:
        return False
    import optimizers_b200
    from optimizers_b200 import config

    for name in _ALIASED:
        module = types.ModuleType(name)
        module.__ob200_alias__ = True  # type: ignore[attr-defined]
        source = optimizers_b200 if name == "distributed_shampoo" else config
        for attr in dir(source):
            if not attr.startswith("_"):
                setattr(module, attr, getattr(source, attr))
        if name in ("distributed_shampoo", "distributed_shampoo.preconditioner"):
            module.__path__ = []  # type: ignore[attr-defined]  # a package, so that sub-module paths resolve
        sys.modules[name] = module
    sys.modules["distributed_shampoo"].shampoo_types = sys.modules["distributed_shampoo.shampoo_types"]  # type: ignore[attr-defined]
    sys.modules["distributed_shampoo"].preconditioner = sys.modules["distributed_shampoo.preconditioner"]  # type: ignore[attr-defined]
    sys.modules["distributed_shampoo.preconditioner"].matrix_functions_types = sys.modules[  # type: ignore[attr-defined]
        "distributed_shampoo.preconditioner.matrix_functions_types"
    ]
    return True
