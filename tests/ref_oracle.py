"""Access to the unmodified reference library (installed under baseline/_ref) as a test oracle."""

import importlib
import os
import sys

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


def reference_available() -> bool:
    return os.path.isdir(os.path.join(REF_DIR, "distributed_shampoo"))


def reference():
    """The reference's ``distributed_shampoo`` package."""
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module("distributed_shampoo")
