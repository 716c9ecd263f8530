"""ctypes binding of libhkb.so, the C-ABI CUDA library (include/hkb.h).

The reference reaches its device code through ctypes as well (HIP's module API,
python/hk/runtime/codeobj.py:87-113); here the thing bound is one prebuilt shared
library instead of a per-kernel code object. There is no fallback: if the library
is missing or does not load, `load()` raises and every op built on it raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path
from typing import Optional

LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libhkb.so"

KV_BF16 = 0
KV_FP8_E4M3 = 1
KV_F16 = 2          # float16 throughout: cache, new rows, query and output
MAX_SPLITS = 256
MAX_GROUP = 16
STATIC_SCRATCH_BYTES = 8 << 20
ERR_STATIC_SCRATCH = -12
ERR_CUDA = -100


class CacheT(Structure):
    """hkb_cache_t: base pointer + element strides of one paged cache tensor."""

    _fields_ = [("ptr", c_void_p), ("stride_block", c_int64), ("stride_token", c_int64),
                ("stride_head", c_int64), ("num_blocks", c_int64)]


class ExchangeT(Structure):
    """hkb_exchange_t: every rank's gather buffer and state block as mapped in this process."""

    _fields_ = [("world", c_int), ("rank", c_int), ("gather", c_void_p * 8), ("state", c_void_p * 8)]


class HkbError(RuntimeError):
    """A refused or failed hkb call; `.code` is the hkb_status."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn}: {text} (hkb status {code})")
        self.code = code


#: every symbol include/hkb.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "hkb_reshape_and_cache": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, CacheT, CacheT,
                                      c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                      c_void_p]),
    "hkb_paged_decode": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, CacheT, CacheT,
                                 c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                 c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                 c_void_p]),
    "hkb_paged_decode_xsplit": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                                        c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                        c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "hkb_paged_decode_ablate": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, CacheT, CacheT,
                                        c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_int, c_void_p]),
    "hkb_paged_decode_static": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, CacheT, CacheT,
                                        c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "hkb_decode_step": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                                c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int,
                                CacheT, CacheT, c_void_p, c_int64, c_int, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
                                c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "hkb_decode_step_record": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                       c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int,
                                       CacheT, CacheT, c_void_p, c_int64, c_int, c_void_p, c_void_p,
                                       c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
                                       c_int, c_void_p, c_void_p, c_void_p]),
    "hkb_exchange_gather_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "hkb_exchange_state_bytes": (c_size_t, []),
    "hkb_kvsplit_push": (c_int, [ExchangeT, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "hkb_kvsplit_merge": (c_int, [ExchangeT, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "hkb_exchange_state_bytes_rows": (c_size_t, [c_int, c_int]),
    "hkb_kvsplit_exchange": (c_int, [ExchangeT, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int,
                                     c_int, c_int, c_int, c_int, c_void_p]),
    "hkb_arrivals_bytes": (c_size_t, [c_int, c_int]),
    "hkb_paged_prefill": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, CacheT, CacheT,
                                  c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "hkb_paged_prefill_trace": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, CacheT, CacheT,
                                        c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                        c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p,
                                        c_void_p]),
    "hkb_prefill_tile_rows": (c_int, [c_int, c_int]),
    "hkb_prefill_uses_tcgen05": (c_int, [c_int, c_int]),
    "hkb_prefill_tc_error": (c_int, [c_int]),
    "hkb_merge": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p,
                          c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "hkb_walk_uses_mma": (c_int, [c_int, c_int]),
    "hkb_plan_splits": (c_int, [c_int, c_int, c_int, c_int]),
    "hkb_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "hkb_scratch_lse_offset": (c_size_t, [c_int, c_int, c_int, c_int]),
    "hkb_hbm_read_probe": (c_int, [c_void_p, c_size_t, c_int, c_int, c_void_p, c_void_p]),
    "hkb_sm_count": (c_int, [c_int]),
    "hkb_strerror": (c_char_p, [c_int]),
    "hkb_last_cuda_error": (c_int, []),
    "hkb_version": (c_int, []),
}

_LIB: Optional[ctypes.CDLL] = None


def load(path: Optional[os.PathLike] = None) -> ctypes.CDLL:
    """The loaded library with every entry point typed. Raises if it is not built."""
    global _LIB
    if _LIB is not None and path is None:
        return _LIB
    p = Path(path) if path is not None else Path(os.environ.get("HKB_LIB") or LIB_PATH)
    if not p.exists():
        raise ImportError(
            f"{p} is not built. Build it with `python -m hk_dsl_b200.csrc.build` (nvcc, sm_100a); "
            f"there is no CPU or PyTorch fallback for the paged KV path.")
    lib = ctypes.CDLL(str(p))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError names a missing symbol
        fn.restype = res
        fn.argtypes = args
    if path is None:
        _LIB = lib
    return lib


def strerror(code: int) -> str:
    return load().hkb_strerror(code).decode()


def check(fn: str, code: int) -> None:
    """Raise HkbError for a non-zero status."""
    if code == 0:
        return
    text = strerror(code)
    if code == ERR_CUDA:
        text += f": cudaError {load().hkb_last_cuda_error()}"
    raise HkbError(fn, code, text)
