"""The vLLM plugin entry point: decide which routes are on, apply them, say so in one line.

vLLM V1 runs the model in a spawned EngineCore process, so a patch applied in the caller
never reaches it; a `vllm.general_plugins` entry point runs in every process
(python/hk/integration/_vllm_plugin.py:3-14, 145-216 of the reference). `register()` never
raises: a plugin that throws takes the engine's startup with it, and a route that did not
apply is a slower server, not a broken one. Before a route is applied its engine contract is
checked (`contract.py`: the names and parameters it binds to still exist); a route whose
contract is broken, or whose `apply` raises, stays off with its own warning line and the
other proceeds.

    [project.entry-points."vllm.general_plugins"]
    hk = "hk_dsl_b200.integration._vllm_plugin:register"
"""

from __future__ import annotations

import os
from typing import Callable, Dict, Tuple


def _backend() -> Tuple[str, Callable]:
    from . import switches, vllm_backend

    slot = switches.value("vllm_backend") or None
    return vllm_backend.register(slot), (lambda: None)


def _prefill() -> Tuple[str, Callable]:
    from . import vllm_prefill

    return vllm_prefill.apply(), vllm_prefill.revert


#: route -> its apply, returning (report, revert); in the order they are applied
APPLY: Dict[str, Callable[[], Tuple[str, Callable]]] = {"vllm_backend": _backend, "vllm_prefill": _prefill}

REVERT: Dict[str, Callable] = {}


def register() -> None:
    from . import switches

    pid = os.getpid()
    if switches.disabled():
        print(f"[hk] vLLM: off ({switches.DISABLE}=1), stock (pid {pid})", flush=True)
        return
    try:
        from ..runtime import lib

        lib.load()
    except Exception as e:  # noqa: BLE001 -- no library: every route stays off, the engine is stock
        print(f"[hk] vLLM: off (the hkb library did not load: {type(e).__name__}: {e}), stock (pid {pid})",
              flush=True)
        return
    routes = switches.on("vllm")
    if not routes:
        why = switches.decide("vllm_prefill").why
        print(f"[hk] vLLM: no route on ({why}), stock (pid {pid})", flush=True)
        return
    # each route's engine contract first (introspection only); a route whose contract is broken, or
    # whose apply raises, stays off with its own warning line and the other proceeds
    from . import contract

    notes, done, off = contract.apply_routes(routes, APPLY)
    REVERT.update(done)
    applied = list(done)
    if not applied:
        print(f"[hk] vLLM: no route applied ({len(off)} off, see the warnings), stock (pid {pid})", flush=True)
        return
    on = ", ".join(f"{n} ({d.why})" for n, d in routes.items() if n in applied)
    left = f"; OFF: {', '.join(off)}" if off else ""
    print(f"[hk] vLLM routes on: {on}{left}; {'; '.join(notes)} (pid {pid})", flush=True)
