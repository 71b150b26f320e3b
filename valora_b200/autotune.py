"""Measure the tile table on the GPU at hand and write valora_b200/tile_table.json.

    python -m valora_b200.autotune [--out PATH] [--reps N] [--quick]

What is swept (one B200, CUDA events, medians over --reps steps after warm-up):

* steps whose ranks stay <= 64 (the mixed prefill + decode batch, rank 64, seven
  projection shapes): stages of the shrink ring (2 / 3 / 4) and of the expand
  ring (3 / 4), each kernel picked by its own time;
* steps that may meet rank 128 (the prefill batch with ranks 8..128 and the
  1024-adapter decode-heavy batch): shrink ring 2 / 3 stages (a rank-128 K block
  of a full tile does not fit a 48 KB stage; the expand needs its 64 KB stages);
* single drop-in calls (the six-segment fp16 case, ranks 8..32, and the same
  segments at rank 128): shrink ring, expand ring, and the row count of the
  tiles a shrink with few rows is cut into (32 / 64 / 128);
* engine thresholds: the run length from which consecutive rows go to 128-row
  tiles instead of gather tiles (8 / 16 / 32) and the smallest resident rank
  below which a gather tile of the expand uses the wide stage form (decided per
  tile; never / < 17 / < 33 / < 65 / all), on the decode-heavy batch with all
  adapters at rank 16, 32, 64 and 128; and the rows per gather tile (16 / 32).

The reference's counterpart is the table shape_to_config in
valora/models/peft/lora_unordered_batch_infer.py:25-172 (six CUTLASS tile
integers per shape, measured offline on an Ampere part).
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from . import _lib, ops, tile_table, workloads
from .microbench import _time_walk
from .pool import AdapterPool


def _entries(step64, step128, call64, call128):
    return [dict(max_rank=64, step=1, **step64), dict(max_rank=128, step=1, **step128),
            dict(max_rank=64, step=0, **call64), dict(max_rank=128, step=0, **call128)]


def _step_ms(batch, layers, reps, dev, engine_kw=None):
    """Median (shrink ms, expand ms, step ms) of LoraStepEngine.step on `batch`."""
    from .engine import LoraStepEngine
    batch.layers = layers
    eng = LoraStepEngine(batch.projections, batch.ranks, batch.scalings(), batch.dtype, dev, layers, batch.T,
                         **(engine_kw or {}))
    eng.randomize_weights(seed=batch.seed)
    g = torch.Generator(device=dev)
    g.manual_seed(batch.seed + 7919)
    for l in range(layers):
        for p in range(len(batch.projections)):
            eng.x[l][p].normal_(generator=g)
            eng.y[l][p].normal_(generator=g)
    tok = torch.from_numpy(batch.tok_adapter.astype(np.int64)).to(dev)
    for _ in range(3):
        eng.step(tok)
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        eng.step_timed(tok, ev)
        torch.cuda.synchronize()
        out.append((ev[1].elapsed_time(ev[2]), ev[2].elapsed_time(ev[3]), ev[0].elapsed_time(ev[3])))
    if ops.device_status() != 0:
        raise SystemExit("a kernel reported a status while tuning")
    del eng
    torch.cuda.empty_cache()
    return tuple(float(np.median([o[i] for o in out])) for i in range(3))


def _call_us(ranks, reps, dev, layers=16):
    """Median (shrink us, expand us) of one drop-in vlr_atmm call over the six-segment batch."""
    b = workloads.config0()
    H, n_ad, T = workloads.H, b.n_adapters, b.T
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    pools_a = [AdapterPool(sum(ranks) + 16, H, 1, b.dtype, dev, 1) for _ in range(layers)]
    pools_b = [AdapterPool(sum(ranks) + 16, H, 1, b.dtype, dev, 1) for _ in range(layers)]
    for pools in (pools_a, pools_b):
        for pool in pools:
            for a in range(n_ad):
                pool.load_adapter(f"a{a}", ranks[a], 1.0, [[None]])
            pool.buffer[0].copy_((torch.randn(pool.buffer[0].shape, generator=g, device=dev) * 0.02).to(b.dtype))
    x = [torch.randn(T, H, generator=g, device=dev).to(b.dtype) for _ in range(layers)]
    y = [torch.randn(T, H, generator=g, device=dev).to(b.dtype) for _ in range(layers)]
    v = [torch.zeros(T, max(ranks), dtype=b.dtype, device=dev) for _ in range(layers)]
    idx = torch.from_numpy(b.tok_adapter.astype(np.int64)).to(dev)
    packer = ops.Packer(T, n_ad, dev)
    pk = packer.pack(idx, pools_a[0].a_len, sort=False)
    P = pk.host_counts()["P"]
    tables = (pk.seg_len, pk.seg_rank, pk.seg_adapter, pk.seg_start)
    wv = lambda pool: pool.buffer[0].view(pool.buffer[0].shape[0], 32, H // 32)
    wa, wb = [wv(p) for p in pools_a], [wv(p) for p in pools_b]
    sc = pools_a[0].a_scaling

    def shrink(l):
        p = pools_a[l]
        ops.atmm(v[l], x[l], wa[l], p.a_start, p.a_len, p.a_loc, idx, 0, sc, *tables, None, P)

    def expand(l):
        p = pools_b[l]
        ops.atmm(y[l], v[l], wb[l], p.a_start, p.a_len, p.a_loc, idx, 0, sc, *tables, None, P, apply_scale=True)

    return (_time_walk(shrink, layers, reps, 2) * 1e3 / layers, _time_walk(expand, layers, reps, 2) * 1e3 / layers)


def _all_ranks(batch, r):
    batch.ranks = np.full_like(batch.ranks, r)
    return batch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=tile_table.DEFAULT_PATH)
    ap.add_argument("--reps", type=int, default=8)
    ap.add_argument("--quick", action="store_true", help="fewer copies per measurement")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("autotune needs a CUDA device")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = _lib.load()
    base = json.loads(json.dumps(tile_table.BUILTIN))
    s64 = dict(shrink_stages=4, expand_stages=4, small_call_rows=32, wide_gather_below_rank=33)
    s128 = dict(shrink_stages=3, expand_stages=3, small_call_rows=32, wide_gather_below_rank=33)
    c64, c128 = dict(s64), dict(s128)
    log = {}

    def use(**kw):
        base["entries"] = _entries(kw.get("s64", s64), kw.get("s128", s128), kw.get("c64", c64), kw.get("c128", c128))
        tile_table.apply(lib, base)

    L3, L2, L4 = (2, 2, 4) if args.quick else (4, 4, 8)
    # ---- steps, rank <= 64: shrink and expand stages, each by its own kernel time
    res = {}
    for ss, es in ((4, 4), (3, 3), (2, 4)):
        use(s64=dict(shrink_stages=ss, expand_stages=es, small_call_rows=32, wide_gather_below_rank=33))
        res[(ss, es)] = _step_ms(workloads.config3(), L3, args.reps, dev)
    shrink_ms = {4: res[(4, 4)][0], 3: res[(3, 3)][0], 2: res[(2, 4)][0]}
    expand_ms = {4: res[(4, 4)][1], 3: res[(3, 3)][1]}
    s64 = dict(shrink_stages=min(shrink_ms, key=shrink_ms.get), expand_stages=min(expand_ms, key=expand_ms.get),
               small_call_rows=32, wide_gather_below_rank=33)
    log["step_rank64"] = {"workload": f"cfg3 x {L3} layers", "shrink_ms_by_stages": shrink_ms, "expand_ms_by_stages": expand_ms}
    # ---- steps that may meet rank 128
    shrink_ms = {}
    for ss in (3, 2):
        use(s128=dict(shrink_stages=ss, expand_stages=3, small_call_rows=32, wide_gather_below_rank=33))
        a = _step_ms(workloads.config2(), L2, args.reps, dev)
        b = _step_ms(workloads.config4(), L4, args.reps, dev)
        shrink_ms[ss] = a[0] + b[0]
    s128 = dict(shrink_stages=min(shrink_ms, key=shrink_ms.get), expand_stages=3, small_call_rows=32,
                wide_gather_below_rank=33)
    log["step_rank128"] = {"workload": f"cfg2 x {L2} + cfg4 x {L4}", "shrink_ms_by_stages": shrink_ms}
    # ---- single calls
    for name, ranks, stages_s, stages_e in (("call_rank64", [8, 16, 16, 32], (4, 3, 2), (4, 3)),
                                            ("call_rank128", [128, 128, 128, 128], (3, 2), (3,))):
        best_s, best_e, rec = None, None, {}
        for ss in stages_s:
            for rows in (32, 64, 128):
                ch = dict(shrink_stages=ss, expand_stages=stages_e[0], small_call_rows=rows, wide_gather_below_rank=33)
                use(**({"c64": ch} if name == "call_rank64" else {"c128": ch}))
                us = _call_us(ranks, args.reps, dev)[0]
                rec[f"shrink stages {ss} rows {rows}"] = us
                if best_s is None or us < best_s[0]:
                    best_s = (us, ss, rows)
        for es in stages_e:
            ch = dict(shrink_stages=best_s[1], expand_stages=es, small_call_rows=best_s[2], wide_gather_below_rank=33)
            use(**({"c64": ch} if name == "call_rank64" else {"c128": ch}))
            us = _call_us(ranks, args.reps, dev)[1]
            rec[f"expand stages {es}"] = us
            if best_e is None or us < best_e[0]:
                best_e = (us, es)
        ch = dict(shrink_stages=best_s[1], expand_stages=best_e[1], small_call_rows=best_s[2],
                  wide_gather_below_rank=33)
        if name == "call_rank64":
            c64 = ch
        else:
            c128 = ch
        log[name] = {"workload": f"six segments, 928 rows, ranks {ranks}", "us_per_call": rec}
    use()
    # ---- engine thresholds on the decode-heavy batch
    eng_log = {}
    best_min, best_ms = 16, None
    for mm in (8, 16, 32):
        ms = _step_ms(workloads.config4(), L4, args.reps, dev, dict(mma_min_rows=mm))[2] + \
            _step_ms(workloads.config3(), L3, args.reps, dev, dict(mma_min_rows=mm))[2]
        eng_log[f"mma_min_rows {mm}"] = ms
    best_min, best_ms = 16, eng_log["mma_min_rows 16"]
    for mm in (8, 32):                                   # another value only if it is clearly (1 %) better
        if eng_log[f"mma_min_rows {mm}"] < 0.99 * best_ms:
            best_min, best_ms = mm, eng_log[f"mma_min_rows {mm}"]
    wide = {}
    for r in (16, 32, 64, 128):
        off = _step_ms(_all_ranks(workloads.config4(), r), L4, args.reps, dev, dict(wide_gather=False))[1]
        on = _step_ms(_all_ranks(workloads.config4(), r), L4, args.reps, dev, dict(wide_gather=True))[1]
        wide[r] = {"plain_ms": off, "wide_ms": on}
    below = 0
    for r in (16, 32, 64, 128):
        if wide[r]["wide_ms"] < wide[r]["plain_ms"]:
            below = r + 1
        else:
            break
    eng_log["expand_ms_by_rank"] = wide
    for e in (s64, s128, c64, c128):
        e["wide_gather_below_rank"] = below
    rows_ms = {}
    for gr in (16, 32):
        rows_ms[gr] = _step_ms(workloads.config4(), L4, args.reps, dev, dict(gather_rows_per_tile=gr))[2] + \
            _step_ms(workloads.config3(), L3, args.reps, dev, dict(gather_rows_per_tile=gr))[2]
    best_rows = min(rows_ms, key=rows_ms.get)
    eng_log["step_ms_by_gather_rows"] = rows_ms
    table = {
        "gpu": torch.cuda.get_device_name(dev),
        "how": "python -m valora_b200.autotune (CUDA events, medians; see the module docstring for what is swept)",
        "entries": _entries(s64, s128, c64, c128),
        "engine": {"mma_min_rows": best_min, "gather_rows_per_tile": best_rows},
        "measurements": {**log, "engine": eng_log},
    }
    with open(args.out, "w") as f:
        json.dump(table, f, indent=1)
    tile_table.apply(lib, table)
    print(json.dumps({"written": args.out, "entries": table["entries"], "engine": table["engine"]}))


if __name__ == "__main__":
    main()
