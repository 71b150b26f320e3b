"""The measured tile table: launch-level choices of the tensor-core kernels per
kind of call and rank bound, plus the engine-level thresholds that go with them.

The reference keeps a table of six CUTLASS tile integers per (adapters, first
sequence length, K, N), measured on an Ampere part
(valora/models/peft/lora_unordered_batch_infer.py:25-172, looked up in
get_config_a / get_config_b, :216-236).  Here `tile_table.json` (written by
`python -m valora_b200.autotune` on the GPU it names) holds, per (step or single
call, rank bound): how the operand ring is cut into stages for the shrink and
for the expand, and the row count of a small drop-in shrink's tiles; and for
the expand, below which adapter rank a gather tile uses the wide stage form;
for the engine: from which consecutive-run length rows go to 128-row tiles
instead of gather tiles, and how many rows a gather tile takes.  The library gets the launch-level part through
vlr_set_tile_table when it is loaded; VLR_TILE_TABLE=<path> names another file.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_PATH = os.path.join(HERE, "tile_table.json")

# what the library falls back to without a table (its built-in entries), and the engine defaults
BUILTIN = {
    "gpu": None,
    "entries": [
        {"max_rank": 64, "step": 1, "shrink_stages": 4, "expand_stages": 4, "small_call_rows": 32,
         "wide_gather_below_rank": 33},
        {"max_rank": 128, "step": 1, "shrink_stages": 3, "expand_stages": 3, "small_call_rows": 32,
         "wide_gather_below_rank": 33},
        {"max_rank": 64, "step": 0, "shrink_stages": 4, "expand_stages": 4, "small_call_rows": 32,
         "wide_gather_below_rank": 33},
        {"max_rank": 128, "step": 0, "shrink_stages": 3, "expand_stages": 3, "small_call_rows": 32,
         "wide_gather_below_rank": 33},
    ],
    "engine": {"mma_min_rows": 16, "gather_rows_per_tile": 32},
}


class _Choice(ctypes.Structure):
    _fields_ = [("max_rank", ctypes.c_int32), ("step", ctypes.c_int32), ("shrink_stages", ctypes.c_int32),
                ("expand_stages", ctypes.c_int32), ("small_call_rows", ctypes.c_int32),
                ("wide_gather_below_rank", ctypes.c_int32)]


_current = None


def path() -> str:
    return os.environ.get("VLR_TILE_TABLE") or DEFAULT_PATH


def load(p: Optional[str] = None) -> dict:
    """The table in force: the file if there is one, else the built-in choices."""
    p = p or path()
    if os.path.exists(p):
        with open(p) as f:
            t = json.load(f)
        t.setdefault("engine", dict(BUILTIN["engine"]))
        for k, v in BUILTIN["engine"].items():
            t["engine"].setdefault(k, v)
        return t
    if os.environ.get("VLR_TILE_TABLE"):
        raise RuntimeError(f"VLR_TILE_TABLE names a file that does not exist: {p}")
    return json.loads(json.dumps(BUILTIN))


def apply(lib, table: Optional[dict] = None) -> dict:
    """Hand the launch-level entries to the library; returns the table in force."""
    global _current
    t = table if table is not None else load()
    ent = t["entries"]
    arr = (_Choice * max(len(ent), 1))()
    for i, e in enumerate(ent):
        arr[i] = _Choice(int(e["max_rank"]), int(e["step"]), int(e["shrink_stages"]), int(e["expand_stages"]),
                         int(e["small_call_rows"]), int(e.get("wide_gather_below_rank", 33)))
    rc = lib.vlr_set_tile_table(ctypes.cast(arr, ctypes.c_void_p), len(ent))
    if rc != 0:
        raise RuntimeError(f"vlr_set_tile_table refused the table (code {rc}): {ent}")
    _current = t
    return t


def current() -> dict:
    return _current if _current is not None else load()


def choice(lib, step: bool, max_rank: int) -> dict:
    """What the launcher will do for a launch of this kind and rank bound."""
    c = _Choice()
    rc = lib.vlr_get_tile_choice(1 if step else 0, int(max_rank), ctypes.byref(c))
    if rc != 0:
        raise RuntimeError(f"vlr_get_tile_choice failed (code {rc})")
    return {"max_rank": c.max_rank, "step": c.step, "shrink_stages": c.shrink_stages,
            "expand_stages": c.expand_stages, "small_call_rows": c.small_call_rows,
            "wide_gather_below_rank": c.wide_gather_below_rank}
