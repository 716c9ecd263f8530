"""Which of the engine routes of this build are on, decided from environment variables.

The same switches, values and precedence as hk-dsl's `hk.integration.switches`
(python/hk/integration/switches.py:10-24, 286-350), for the two routes this build carries:
the decoder attention backend (`vllm_backend`, `HK_VLLM_BACKEND`, off until asked for) and
the in-place attention route (`vllm_prefill`, `HK_VLLM_PREFILL`, on by default on a GPU it
was validated on -- here B200, `sm_100`).

The first rule that applies decides:

1. `HK_DISABLE` set to anything but an off word turns every route off.
2. The engine's switch (`HK_PATCH_VLLM`) set to an off word turns the engine's routes off.
3. The route's own switch: an off word turns it off; anything else turns it on, and a value
   that is not a plain on word is kept (`HK_VLLM_BACKEND=<slot>`).
4. The route's default, which applies only on a validated arch.

An empty value is unset. Off words: 0, off, no, false. On words: 1, on, yes, true, all.
This module imports nothing but the standard library, so it loads without torch or a GPU.

    python -m hk_dsl_b200.integration --status
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Tuple

OFF = ("0", "off", "no", "false")
ON = ("1", "on", "yes", "true", "all")

DISABLE = "HK_DISABLE"

#: engine -> the switch that turns all of its routes off
ENGINES: Dict[str, str] = {"vllm": "HK_PATCH_VLLM", "sglang": "HK_PATCH_SGLANG", "ops": ""}

#: the arch name this build's kernels are validated on
SM100 = "sm_100"


@dataclass(frozen=True)
class Route:
    name: str
    engine: str
    env: str
    default: bool
    arches: Tuple[str, ...]
    what: str
    evidence: str


@dataclass(frozen=True)
class Decision:
    on: bool
    why: str
    value: str = ""


ROUTES: Dict[str, Route] = {r.name: r for r in (
    Route("vllm_backend", "vllm", "HK_VLLM_BACKEND", False, (),
          "the decoder's paged attention backend: cache write + paged GQA decode (bf16 and fp8-e4m3 KV)",
          "off: it replaces the engine's decoder attention for every model. It raises, rather than falls "
          "back, on sliding windows, sinks, softcap, ALiBi, fp16 and other head sizes; batches with "
          "prefill in them are not built yet"),
    Route("vllm_prefill", "vllm", "HK_VLLM_PREFILL", True, (SM100,),
          "decode-only attention calls in place on the engine's own cache (unified_attention, "
          "chunked_prefill_paged_decode); cache write and block size stay the engine's; any other call "
          "falls back to the engine's kernel and is counted",
          "parity with the float64 reference on every GQA shape, page size and layout of the test suite; "
          "KV read at 75-95% of measured HBM bandwidth on B200"),
)}


def _setting(env: Mapping[str, str], var: str) -> str:
    """A variable's value with blanks trimmed; unset, empty and "no such variable" are all ""."""
    return str(env.get(var, "")).strip() if var else ""


def is_off(v: str) -> bool:
    return v.strip().lower() in OFF


def disabled(env: Optional[Mapping[str, str]] = None) -> bool:
    """Whether HK_DISABLE turns everything off."""
    setting = _setting(os.environ if env is None else env, DISABLE)
    return setting != "" and not is_off(setting)


_ARCH_SEEN: Dict[str, Optional[str]] = {}


def arch() -> Optional[str]:
    """`sm_<major><minor>` of the current GPU (`sm_100` on a B200), `HK_ARCH` if set, or None
    without a GPU: a default never assumes one. The GPU is asked once a process."""
    override = os.environ.get("HK_ARCH", "").strip()
    if override:
        return override
    if "gpu" not in _ARCH_SEEN:
        name = None
        try:
            import torch  # noqa: PLC0415

            if torch.cuda.is_available():
                name = "sm_%d%d" % torch.cuda.get_device_capability()
        except Exception:  # noqa: BLE001 -- no torch, no driver: nothing is validated here
            name = None
        _ARCH_SEEN["gpu"] = name
    return _ARCH_SEEN["gpu"]


# ---- the rules, in order of precedence. Each looks at one thing and either settles the
# ---- question (a Decision) or passes (None); `decide` returns the first answer.

def _rule_kill_switch(route: Route, env: Mapping[str, str], gpu) -> Optional[Decision]:
    if disabled(env):
        return Decision(False, f"{DISABLE}={_setting(env, DISABLE)}")
    return None


def _rule_engine_switch(route: Route, env: Mapping[str, str], gpu) -> Optional[Decision]:
    var = ENGINES.get(route.engine, "")
    setting = _setting(env, var)
    if setting and is_off(setting):
        return Decision(False, f"{var}={setting}")
    return None


def _rule_route_switch(route: Route, env: Mapping[str, str], gpu) -> Optional[Decision]:
    setting = _setting(env, route.env)
    if not setting:
        return None
    said = f"{route.env}={setting}"
    if is_off(setting):
        return Decision(False, said)
    # on; a value that is not a plain on word rides along (a backend slot name, say)
    return Decision(True, said, setting if setting.lower() not in ON else "")


def _rule_default(route: Route, env: Mapping[str, str], gpu) -> Optional[Decision]:
    if not route.default:
        return Decision(False, "default off")
    found = arch() if gpu == "detect" else gpu
    if found in route.arches:
        return Decision(True, f"default on ({found})")
    return Decision(False, f"default off on {found or 'no GPU'} (validated on {', '.join(route.arches)})")


RULES = (_rule_kill_switch, _rule_engine_switch, _rule_route_switch, _rule_default)


def decide(name: str, env: Optional[Mapping[str, str]] = None, gpu: Optional[str] = "detect") -> Decision:
    """On or off for one route, and which rule decided."""
    route = ROUTES[name]
    env = os.environ if env is None else env
    for rule in RULES:
        verdict = rule(route, env, gpu)
        if verdict is not None:
            return verdict
    raise AssertionError("the default rule always decides")


def enabled(name: str, env: Optional[Mapping[str, str]] = None) -> bool:
    return decide(name, env).on


def value(name: str, env: Optional[Mapping[str, str]] = None) -> str:
    """A route's explicit value (a slot name), or "" for plain on."""
    return decide(name, env).value


def routes(engine: str) -> List[Route]:
    return [route for route in ROUTES.values() if route.engine == engine]


def on(engine: str, env: Optional[Mapping[str, str]] = None) -> Dict[str, Decision]:
    """Every route of `engine` that is on: name -> its decision."""
    verdicts = {route.name: decide(route.name, env) for route in routes(engine)}
    return {name: verdict for name, verdict in verdicts.items() if verdict.on}


def table(env: Optional[Mapping[str, str]] = None) -> str:
    """Every route, on or off and why: what `--status` prints."""
    verdicts = {name: decide(name, env) for name in ROUTES}
    name_w = max(map(len, ROUTES))
    env_w = max(len(route.env) for route in ROUTES.values())
    lines = []
    for name, verdict in verdicts.items():
        state = "on" if verdict.on else "off"
        lines.append(f"{name.ljust(name_w)}  {ROUTES[name].env.ljust(env_w)}  {state.ljust(3)}  {verdict.why}")
    return "\n".join(lines)
