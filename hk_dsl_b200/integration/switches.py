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


def _get(env: Mapping[str, str], name: str) -> str:
    return env.get(name, "").strip() if name else ""


def is_off(v: str) -> bool:
    return v.strip().lower() in OFF


def disabled(env: Optional[Mapping[str, str]] = None) -> bool:
    """Whether HK_DISABLE turns everything off."""
    v = _get(os.environ if env is None else env, DISABLE)
    return bool(v) and not is_off(v)


_ARCH: List[Optional[str]] = []


def arch() -> Optional[str]:
    """`sm_<major><minor>` of the current GPU (`sm_100` on a B200), `HK_ARCH` if set, or None
    without a GPU: a default never assumes one."""
    forced = os.environ.get("HK_ARCH", "").strip()
    if forced:
        return forced
    if not _ARCH:
        found = None
        try:
            import torch  # noqa: PLC0415

            if torch.cuda.is_available():
                major, minor = torch.cuda.get_device_capability()
                found = f"sm_{major}{minor}"
        except Exception:  # noqa: BLE001 -- no torch, no driver: nothing is validated here
            found = None
        _ARCH.append(found)
    return _ARCH[0]


def decide(name: str, env: Optional[Mapping[str, str]] = None, gpu: Optional[str] = "detect") -> Decision:
    """On or off for one route, and which rule decided."""
    env = os.environ if env is None else env
    r = ROUTES[name]
    if disabled(env):
        return Decision(False, f"{DISABLE}={_get(env, DISABLE)}")
    master = ENGINES.get(r.engine, "")
    mv = _get(env, master)
    if mv and is_off(mv):
        return Decision(False, f"{master}={mv}")
    v = _get(env, r.env)
    if v:
        if is_off(v):
            return Decision(False, f"{r.env}={v}")
        return Decision(True, f"{r.env}={v}", "" if v.lower() in ON else v)
    if not r.default:
        return Decision(False, "default off")
    here = arch() if gpu == "detect" else gpu
    if here in r.arches:
        return Decision(True, f"default on ({here})")
    return Decision(False, f"default off on {here or 'no GPU'} (validated on {', '.join(r.arches)})")


def enabled(name: str, env: Optional[Mapping[str, str]] = None) -> bool:
    return decide(name, env).on


def value(name: str, env: Optional[Mapping[str, str]] = None) -> str:
    """A route's explicit value (a slot name), or "" for plain on."""
    return decide(name, env).value


def routes(engine: str) -> List[Route]:
    return [r for r in ROUTES.values() if r.engine == engine]


def on(engine: str, env: Optional[Mapping[str, str]] = None) -> Dict[str, Decision]:
    """Every route of `engine` that is on: name -> its decision."""
    found = {}
    for r in routes(engine):
        d = decide(r.name, env)
        if d.on:
            found[r.name] = d
    return found


def table(env: Optional[Mapping[str, str]] = None) -> str:
    """Every route, on or off and why: what `--status` prints."""
    rows = [(r.name, r.env, "on" if d.on else "off", d.why) for r in ROUTES.values()
            for d in (decide(r.name, env),)]
    w = [max(len(x[i]) for x in rows) for i in range(3)]
    return "\n".join(f"{a:{w[0]}}  {b:{w[1]}}  {c:{w[2]}}  {e}" for a, b, c, e in rows)
