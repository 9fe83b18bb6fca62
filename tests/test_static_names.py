"""Every name a function reads as a global exists in its module (or is a builtin).

The multi-GPU workers, the benchmarks and the error paths of the package run rarely, some only on
a box with several GPUs; a misspelt or left-over name there would show as a ``NameError`` at the
worst time.  ``symtable`` gives, per scope, the names that resolve to module globals; each must be
assigned, imported or defined at module level.
"""

import builtins
import glob
import os
import symtable

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_IMPLICIT = {"__file__", "__name__", "__doc__", "__path__", "__spec__", "__builtins__"}


def _sources():
    files = glob.glob(os.path.join(ROOT, "optimizers_b200", "**", "*.py"), recursive=True)
    files += glob.glob(os.path.join(ROOT, "benchmarks", "*.py")) + glob.glob(os.path.join(ROOT, "tests", "*.py"))
    files += [os.path.join(ROOT, "bench.py"), os.path.join(ROOT, "__graft_entry__.py")]
    return sorted(files)


def _undefined(path):
    source = open(path).read()
    if "import *" in source:
        return []
    top = symtable.symtable(source, path, "exec")
    defined = {s.get_name() for s in top.get_symbols() if s.is_assigned() or s.is_imported() or s.is_namespace()}
    missing = []

    def walk(table):
        for s in table.get_symbols():
            if not s.is_referenced():
                continue
            at_module = table.get_type() == "module" and not (s.is_assigned() or s.is_imported() or s.is_namespace())
            if s.is_global() or at_module:
                name = s.get_name()
                if name not in defined and not hasattr(builtins, name) and name not in _IMPLICIT:
                    missing.append(f"{os.path.relpath(path, ROOT)}: {table.get_name()} reads {name}")
        for child in table.get_children():
            walk(child)

    walk(top)
    return missing


def test_no_function_reads_an_undefined_global():
    files = _sources()
    assert len(files) > 60
    missing = [line for path in files for line in _undefined(path)]
    assert not missing, "\n".join(missing)
