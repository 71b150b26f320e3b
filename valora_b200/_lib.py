"""ctypes binding of libvlr.so.  There is no fallback: if the library is
missing or a symbol is absent, importing the operators fails loudly."""
from __future__ import annotations

import ctypes
import os
import re

from . import build as _build

_HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "vlr.h")

c_i64 = ctypes.c_int64
c_int = ctypes.c_int
c_vp = ctypes.c_void_p
c_sz = ctypes.c_size_t

_SIGS = {
    "vlr_version": (c_int, []),
    "vlr_error_string": (ctypes.c_char_p, [c_int]),
    "vlr_set_device": (c_int, [c_int]),
    "vlr_selftest_bounded_wait": (c_int, [c_i64, c_vp, c_vp, c_vp]),
    "vlr_fused_proj": (c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_i64, c_vp, c_vp, c_i64, c_vp, c_vp, c_i64,
                               c_i64, c_i64, c_i64, c_int, c_vp, c_vp]),
    "vlr_set_tile_table": (c_int, [c_vp, c_int]),
    "vlr_get_tile_choice": (c_int, [c_int, c_int, c_vp]),
    "vlr_device_status": (c_int, [c_int]),
    "vlr_bgmv": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp,
                         c_i64, c_i64, c_i64, c_int, c_int, c_vp]),
    "vlr_atmm": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp,
                         c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64,
                         c_i64, c_i64, c_i64, c_i64, c_int, c_int, c_vp]),
    "vlr_pack_workspace_bytes": (c_sz, [c_i64, c_i64]),
    "vlr_pack": (c_int, [c_vp, c_i64, c_vp, c_i64, c_int, c_int, c_int, c_int,
                         c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "vlr_pack_static": (c_int, [c_vp, c_i64, c_vp, c_i64, c_int, c_int, c_int, c_int,
                                c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp, c_vp, c_vp]),
    "vlr_var_len_copy": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_vp]),
    "vlr_step_plan_bytes": (c_sz, [c_int]),
    "vlr_step_plan_build": (c_int, [c_vp, c_int, c_i64, c_int, c_vp]),
    "vlr_lora_step": (c_int, [c_vp, c_int, c_i64, c_vp, c_vp, c_i64, c_i64, c_vp, c_vp,
                              c_int, c_int, c_int, c_int, c_int, c_vp, c_sz, c_vp, c_vp]),
    "vlr_lora_step_workspace_bytes": (c_sz, [c_i64, c_int]),
}

_lib = None


def declared_symbols():
    """Every function the public header declares."""
    text = open(_HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vlr_[a-z_0-9]+)\s*\(", text)))


def load(build_if_missing: bool = True):
    global _lib
    if _lib is not None:
        return _lib
    trace = os.environ.get("VLR_TRACE") == "1"           # debugging build with the stage trace
    path = _build.LIB_TRACE if trace else _build.LIB
    if not os.path.exists(path):
        if not build_if_missing:
            raise RuntimeError(f"{path} is missing: build it with `python -m valora_b200.build`")
        _build.build(trace=trace)
    lib = ctypes.CDLL(path)
    for name in declared_symbols():
        if not hasattr(lib, name):
            raise RuntimeError(f"libvlr.so does not export {name}")
        if name in _SIGS:
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = _SIGS[name]
    from . import tile_table
    tile_table.apply(lib)                            # the measured launch choices, if a table is committed
    if hasattr(lib, "vlr_debug_set_trace"):          # debug builds (-DVLR_TRACE) only
        lib.vlr_debug_set_trace.restype, lib.vlr_debug_set_trace.argtypes = c_int, [c_vp, c_i64]
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc != 0:
        msg = load().vlr_error_string(rc)
        raise RuntimeError(f"{what} failed: {msg.decode() if msg else rc} (code {rc})")
