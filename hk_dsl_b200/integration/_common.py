"""Rebinding a function in every module that imported it by name.

Replacing `module.fn` reaches callers that go through the module and misses every caller
that did `from module import fn`, which holds its own reference. So a route replaces the
attribute and then walks the already-imported modules under a prefix, rebinding each name
that IS the original object -- by identity, so it needs no knowledge of the engine's version
and cannot touch something that merely has the same name (python/hk/integration/_common.py:26-43
of the reference). `apply()` therefore runs after the engine's modules are imported and
before a model runs.
"""

from __future__ import annotations

import sys
from typing import List, Tuple


def rebind(prefixes: Tuple[str, ...], old, new) -> List[str]:
    """Rebind every attribute of a loaded module under `prefixes` whose value is `old`."""
    done = []
    for mod_name in list(sys.modules):
        mod = sys.modules.get(mod_name)
        if mod is None or not mod_name.startswith(prefixes):
            continue
        try:
            names = [k for k, v in vars(mod).items() if v is old]
        except TypeError:
            continue
        for k in names:
            try:
                setattr(mod, k, new)
            except Exception:  # noqa: BLE001 -- a module that refuses assignment
                continue
            done.append(f"{mod_name}.{k}")
    return done


def importable(name: str) -> bool:
    import importlib.util

    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError):
        return False
