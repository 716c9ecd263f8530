"""The engine contract of the two vLLM routes, checked before a route is applied.

The routes bind to vLLM by name: the backend class subclasses vLLM's attention interfaces and
registers over a slot of its backend enum; the in-place route rebinds `unified_attention` and
`chunked_prefill_paged_decode` and reads their arguments by name. A vLLM release that renames,
moves or re-signs one of those does not make a patch fail loudly -- it makes it route nothing,
or read the wrong argument. So, as the reference does at plugin start
(python/hk/integration/contract.py:1-22, 367-411, 829-906): gather facts about the installed
engine by introspection only (imports, attributes, `inspect.signature`; nothing is launched),
judge them against what each route needs, and leave a route whose contract is broken OFF with
one warning line -- per route, the other one is unaffected.

    python -m hk_dsl_b200.integration.contract        # prints the facts and the verdicts
"""

from __future__ import annotations

import inspect
import json
import os
import sys
from typing import Callable, Dict, Iterable, List, Optional, Tuple

#: The vLLM these routes were run against in this repository's in-engine checks. Another version
#: is not a failure by itself; a broken contract is.
MEASURED_VLLM = "0.22"

#: unified_attention's parameters the stand-in reads (python/hk/integration/vllm_prefill.py:
#: 1068-1095 of the reference reads the same ones)
UNIFIED_NEEDS = ("q", "k", "v", "out", "cu_seqlens_q", "max_seqlen_q", "seqused_k", "softmax_scale", "causal",
                 "block_table")
#: chunked_prefill_paged_decode's
CHUNKED_NEEDS = ("query", "output", "kv_cache_dtype", "key_cache", "value_cache", "block_table", "query_start_loc",
                 "seq_lens", "max_query_len", "k_scale", "v_scale", "sm_scale")
#: attributes of vLLM's attention metadata the backend's forward reads (vllm_backend.py:613-636
#: of the reference; pinned by its tests/hk/engines/test_vllm_contract.py:256-257)
METADATA_NEEDS = ("num_actual_tokens", "slot_mapping", "max_query_len", "block_table", "seq_lens", "query_start_loc",
                  "max_seq_len")
#: AttentionImpl.forward's parameters, in order (vllm_backend.py:613 of the reference)
FORWARD_NEEDS = ("layer", "query", "key", "value", "kv_cache", "attn_metadata", "output")


def names(fn: Callable, drop_self: bool = False) -> List[str]:
    ps = [p.name for p in inspect.signature(fn).parameters.values() if p.kind not in (p.VAR_POSITIONAL, p.VAR_KEYWORD)]
    return ps[1:] if drop_self and ps and ps[0] == "self" else ps


def _expect(ok: bool, problem: str) -> List[str]:
    return [] if ok else [problem]


# ---- the in-place route ------------------------------------------------------------------

def gather_vllm_prefill() -> dict:
    from vllm.v1.attention.ops import chunked_prefill_paged_decode as cpd  # noqa: PLC0415
    from vllm.v1.attention.ops import triton_unified_attention as tua  # noqa: PLC0415

    from . import vllm_prefill  # noqa: PLC0415

    u = vllm_prefill._ORIG_U or tua.unified_attention            # the engine's own, also while patched
    r = vllm_prefill._ORIG_R or cpd.chunked_prefill_paged_decode
    return {"unified_attention": names(u), "chunked_prefill_paged_decode": names(r)}


def judge_vllm_prefill(f: dict) -> List[str]:
    # The stand-ins take vLLM's own signature and read what they need by name; a parameter a newer
    # vLLM adds is refused per call unless it is at its default, so only a LOST name breaks the route.
    lost_u = sorted(set(UNIFIED_NEEDS) - set(f["unified_attention"]))
    lost_r = sorted(set(CHUNKED_NEEDS) - set(f["chunked_prefill_paged_decode"]))
    return (_expect(not lost_u, f"unified_attention lost {lost_u}")
            + _expect(not lost_r, f"chunked_prefill_paged_decode lost {lost_r}"))


# ---- the backend class ---------------------------------------------------------------------

def gather_vllm_backend() -> dict:
    from vllm.v1.attention.backend import AttentionBackend, AttentionImpl  # noqa: PLC0415
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend  # noqa: PLC0415

    facts = {"register_backend": callable(register_backend),
             "backend_slots": [m.name for m in AttentionBackendEnum],
             "impl_forward": names(AttentionImpl.forward, drop_self=True),
             "backend_methods": sorted(n for n in ("get_name", "get_impl_cls", "get_builder_cls", "get_kv_cache_shape",
                                                   "get_supported_head_sizes") if hasattr(AttentionBackend, n))}
    try:
        from vllm.v1.attention.backends.utils import CommonAttentionMetadata  # noqa: PLC0415

        fields = getattr(CommonAttentionMetadata, "__dataclass_fields__", None)
        facts["common_metadata"] = sorted(fields) if fields else sorted(
            n for n in dir(CommonAttentionMetadata) if not n.startswith("_"))
    except Exception as e:  # noqa: BLE001 -- recorded, judged below
        facts["common_metadata"] = f"{type(e).__name__}: {e}"
    return facts


def judge_vllm_backend(f: dict) -> List[str]:
    from . import switches, vllm_backend  # noqa: PLC0415

    slot = switches.value("vllm_backend") or os.environ.get("HK_VLLM_BACKEND_SLOT") or vllm_backend.SLOT
    fwd = list(f["impl_forward"])
    problems = (_expect(f["register_backend"], "vLLM has no register_backend")
                + _expect(slot in f["backend_slots"], f"vLLM's AttentionBackendEnum has no {slot}")
                + _expect(fwd[:len(FORWARD_NEEDS)] == list(FORWARD_NEEDS),
                          f"AttentionImpl.forward now takes {fwd}, the backend passes {list(FORWARD_NEEDS)} in that order")
                + _expect({"get_name", "get_impl_cls", "get_kv_cache_shape"} <= set(f["backend_methods"]),
                          f"AttentionBackend has only {f['backend_methods']}"))
    cm = f.get("common_metadata")
    if isinstance(cm, list):      # the builder reads these from the common metadata
        lost = sorted({"query_start_loc", "seq_lens", "block_table_tensor", "slot_mapping", "num_actual_tokens",
                       "max_query_len"} - set(cm))
        problems += _expect(not lost, f"CommonAttentionMetadata lost {lost}")
    return problems


GATHER: Dict[str, Callable[[], dict]] = {"vllm_prefill": gather_vllm_prefill, "vllm_backend": gather_vllm_backend}
JUDGE: Dict[str, Callable[[dict], List[str]]] = {"vllm_prefill": judge_vllm_prefill, "vllm_backend": judge_vllm_backend}


def check_each(routes: Iterable[str]) -> Dict[str, List[str]]:
    """Each route among `routes` whose contract is broken, with its problems; {} if all hold. A
    module that moved is a broken contract too."""
    broken: Dict[str, List[str]] = {}
    for name in routes:
        if name not in GATHER:
            continue
        try:
            got = JUDGE[name](GATHER[name]())
        except Exception as e:  # noqa: BLE001
            got = [f"{type(e).__name__}: {e}"]
        if got:
            broken[name] = list(got)
    return broken


def engine_version() -> str:
    try:
        import importlib.metadata as md  # noqa: PLC0415

        return f"vllm {md.version('vllm')}"
    except Exception:  # noqa: BLE001
        return "vllm (version unknown)"


def refuse_route(route: str, problems: List[str], what: str = "engine contract FAILED") -> str:
    """The warning line for one route left off (also returned); the other route is unaffected."""
    from . import switches  # noqa: PLC0415

    r = switches.ROUTES.get(route)
    off = f"{r.env}=0" if r is not None else f"{switches.DISABLE}=1"
    line = (f"[hk] WARNING: vLLM: route {route} OFF -- {what} ({engine_version()}; routes run against vllm "
            f"{MEASURED_VLLM}): " + "; ".join(problems) + f". The other route is unaffected. Set {off} to silence "
            f"this. (pid {os.getpid()})")
    print(line, file=sys.stderr, flush=True)
    return line


def apply_routes(routes: Iterable[str], appliers: Dict[str, Callable[[], Tuple[str, Callable]]]
                 ) -> Tuple[List[str], Dict[str, Callable], Dict[str, List[str]]]:
    """Check each route's contract and apply the ones that hold, in `appliers`' order. An applier
    returns (report line, revert). Returns (reports, {applied route: revert}, {route left off: why})."""
    routes = list(routes)
    off = check_each(routes)
    for name, problems in off.items():
        refuse_route(name, problems)
    reports, applied = [], {}
    for name, how in appliers.items():
        if name not in routes or name in off:
            continue
        try:
            report, revert = how()
        except Exception as e:  # noqa: BLE001 -- one route's failure leaves the other on
            off[name] = [f"raised {type(e).__name__}: {e}"]
            refuse_route(name, off[name], "the route failed to apply")
            continue
        reports.append(report)
        applied[name] = revert
    return reports, applied, off


def main(argv: Optional[List[str]] = None) -> int:
    facts, verdicts = {}, {}
    for name in GATHER:
        try:
            facts[name] = GATHER[name]()
            verdicts[name] = JUDGE[name](facts[name])
        except Exception as e:  # noqa: BLE001
            facts[name] = None
            verdicts[name] = [f"{type(e).__name__}: {e}"]
    print(json.dumps({"engine": engine_version(), "facts": facts, "broken": {k: v for k, v in verdicts.items() if v}},
                     indent=1))
    return 1 if any(verdicts.values()) else 0


if __name__ == "__main__":
    sys.exit(main())
