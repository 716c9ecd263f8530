"""python -m hk_dsl_b200.integration --status: every route, on or off, and which rule decided;
the hkb library and the GPU it would run on; the patches' counters in this process."""

from __future__ import annotations

import sys


def status() -> str:
    from . import engine, switches

    lines = [switches.table(), ""]
    try:
        from ..runtime import lib

        lines.append(f"hkb library: {lib.LIB_PATH} (version {lib.load().hkb_version()})")
    except Exception as e:  # noqa: BLE001
        lines.append(f"hkb library: NOT LOADED ({type(e).__name__}: {e})")
    lines.append(f"GPU arch: {switches.arch() or 'no GPU'}")
    for p in engine.PATCHES.values():
        lines.append(p.summary())
    return "\n".join(lines)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if not argv or argv[0] in ("--status", "status"):
        print(status())
        return 0
    print("usage: python -m hk_dsl_b200.integration --status", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
