"""Build libhkb.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m hk_dsl_b200.csrc.build [--force] [--verbose]

No torch headers are involved: the library is plain CUDA runtime + C ABI, so it
cross-compiles on a machine without a GPU and loads through ctypes anywhere.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
LIB_DIR = HERE.parent / "_lib"
LIB = LIB_DIR / "libhkb.so"
STAMP = LIB_DIR / "libhkb.stamp"

SOURCES = ["hkb_api.cu", "hkb_scatter.cu", "hkb_decode.cu", "hkb_prefill.cu", "hkb_probe.cu", "hkb_exchange.cu"]
HEADERS = ["hkb_common.cuh", "hkb_prefill_tc.cuh", "hkb_fold_wide.cuh", "hkb_decode.cuh", "hkb_fold.cuh", "hkb_walk_cc.cuh", "hkb_walk_mma.cuh", "hkb_walk_stream.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-warn-spills",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the hkb library is built with CUDA 12.8+ for sm_100a")
    return exe


def _digest() -> str:
    h = hashlib.sha256()
    for name in SOURCES + HEADERS:
        h.update((HERE / name).read_bytes())
    h.update((ROOT / "include" / "hkb.h").read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def up_to_date() -> bool:
    return LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == _digest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source to an object and link the shared library. Returns its path."""
    if not force and up_to_date():
        return LIB
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose else [])
    procs = []
    for src in SOURCES:
        obj = obj_dir / (src + ".o")
        cmd = [nvcc(), *flags, "-c", str(HERE / src), "-o", str(obj)]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose or "spill" in out.lower() and "0 bytes spill" not in out:
            sys.stderr.write(out)
        objs.append(str(obj))
    cmd = [nvcc(), "-shared", "-o", str(LIB), *objs]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    STAMP.write_text(_digest())
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
