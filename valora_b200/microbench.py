"""Micro-benchmarks on one B200, one JSON line each.

    python -m valora_b200.microbench --config 0     # ragged shrink + expand drop-in call, fp16, 928 tokens in 6 segments
    python -m valora_b200.microbench --config 1     # decode BGMV drop-in call, bf16, 512 tokens
    python -m valora_b200.microbench --config 1 --api step   # the same decode batch through the step API
    python -m valora_b200.microbench --config 2     # prefill, mixed ranks 8..128, fp16, 7 projections (step API)
    python -m valora_b200.microbench --config 3 --shared-x   # the mixed batch with q/k/v and up/gate reading one X each
    VLR_TRACE=1 python -m valora_b200.microbench --config 3 --trace expand   # stage timing of one launch (clock64 stamps
                                                     # of CTA 0; needs the debugging build: python -m valora_b200.build --trace)
    python -m valora_b200.microbench --config 4     # 16384 tokens, 1024 adapters, ranks 16..128, bf16 (step API)

Configs 0 and 1:  A measurement walks `--layers` independent copies
of the operator's tensors (own pools, own activations; together larger than
L2), one shrink and one expand call per copy, and times the walk with CUDA
events on the launching stream; GB/s are algorithmic bytes (activations once,
every touched adapter row once, outputs read + written) over that time.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from . import ops, workloads
from .pool import AdapterPool

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def _time_walk(fn, layers, reps, warmup, eager=False):
    """Median over reps of the device time of one walk over all layers, in ms.
    The walk is captured once into a CUDA graph and replayed, so that what is
    timed is the kernels back to back and not the host's call overhead
    (eager=True launches call by call instead, for profilers)."""
    def walk():
        for l in range(layers):
            fn(l)

    if eager:
        out = []
        for k in range(warmup + reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            walk()
            e1.record()
            torch.cuda.synchronize()
            if k >= warmup:
                out.append(e0.elapsed_time(e1))
        return float(np.median(out))

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            walk()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        walk()
    graph.replay()
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return float(np.median(out))


def bench_bgmv(layers: int, reps: int, warmup: int, dev, eager: bool = False):
    """Config 1 through the 9-argument decode call: shrink (4096 -> 64) then expand
    (64 -> 4096, punica weight layout), per token adapter index, no packing."""
    b = workloads.config1()
    H, r, n_ad, T = 4096, 64, b.n_adapters, b.T
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    pools_a = [AdapterPool(n_ad * r + 16, H, 1, b.dtype, dev, 1) for _ in range(layers)]
    pools_b = [AdapterPool(n_ad * r + 16, H, 1, b.dtype, dev, 1) for _ in range(layers)]
    for pools in (pools_a, pools_b):
        for pool in pools:
            for a in range(n_ad):
                pool.load_adapter(f"a{a}", r, 0.25, [[None]])
            pool.buffer[0].copy_((torch.randn(pool.buffer[0].shape, generator=g, device=dev) * 0.02).to(b.dtype))
    x = [torch.randn(T, H, generator=g, device=dev).to(b.dtype) for _ in range(layers)]
    y = [torch.randn(T, H, generator=g, device=dev).to(b.dtype) for _ in range(layers)]
    v = [torch.zeros(T, r, dtype=b.dtype, device=dev) for _ in range(layers)]
    idx = torch.from_numpy(b.tok_adapter.astype(np.int64)).to(dev)
    pa0 = pools_a[0]
    scales = pa0.a_scaling

    def wview(pool):
        return pool.buffer[0].view(pool.buffer[0].shape[0], 32, H // 32)

    wa = [wview(p) for p in pools_a]
    wb = [wview(p) for p in pools_b]

    def shrink(l):
        p = pools_a[l]
        ops.bgmv(v[l], x[l], wa[l], p.a_start, p.a_len, p.a_loc, idx, 0, scales)

    def expand(l):
        p = pools_b[l]
        ops.bgmv(y[l], v[l], wb[l], p.a_start, p.a_len, p.a_loc, idx, 0, scales)

    touched = len(np.unique(b.tok_adapter))
    e = 2
    bytes_shrink = (T * H + touched * r * H + T * r) * e
    bytes_expand = (T * r + touched * r * H + 2 * T * H) * e
    ms_s = _time_walk(shrink, layers, reps, warmup, eager)
    ms_e = _time_walk(expand, layers, reps, warmup, eager)
    ms_b = _time_walk(lambda l: (shrink(l), expand(l)), layers, reps, warmup, eager)
    if ops.device_status() != 0:
        raise SystemExit("a bounded wait gave up inside a kernel")
    peak, src = _peak()

    def gbs(nbytes, ms):
        return nbytes * layers / (ms * 1e-3) / 1e9

    return {
        "bench": "decode_bgmv_dropin", "workload": b.name, "dtype": "bf16", "tokens": T, "adapters": n_ad,
        "adapters_touched": touched, "rank": r, "hidden": H, "layers_walked": layers,
        "bytes_resident": layers * (2 * (n_ad * r + 16) * H + 2 * T * H) * e,
        "shrink": {"us_per_call": ms_s * 1e3 / layers, "gbs": gbs(bytes_shrink, ms_s),
                   "frac": gbs(bytes_shrink, ms_s) / peak, "algorithmic_bytes": bytes_shrink},
        "expand": {"us_per_call": ms_e * 1e3 / layers, "gbs": gbs(bytes_expand, ms_e),
                   "frac": gbs(bytes_expand, ms_e) / peak, "algorithmic_bytes": bytes_expand},
        "both": {"us_per_pair": ms_b * 1e3 / layers, "gbs": gbs(bytes_shrink + bytes_expand, ms_b),
                 "frac": gbs(bytes_shrink + bytes_expand, ms_b) / peak,
                 "tokens_per_s": T * layers / (ms_b * 1e-3)},
        "peak_gbs": peak, "peak_source": src, "launch": "call by call" if eager else "one CUDA graph per walk, replayed",
    }


def bench_atmm(layers: int, reps: int, warmup: int, dev, eager: bool = False):
    """Config 0 through the 21-argument ragged call: shrink (4096 -> r) then expand
    (r -> 4096) over the six segments, problem table in request order as the
    reference's host packer would build it, adapter scale applied in the expand."""
    b = workloads.config0()
    H, n_ad, T = workloads.H, b.n_adapters, b.T
    ranks = [int(r) for r in b.ranks]
    max_r = max(ranks)
    g = torch.Generator(device=dev)
    g.manual_seed(b.seed)
    pools_a = [AdapterPool(sum(ranks) + 16, H, 1, b.dtype, dev, 1) for _ in range(layers)]
    pools_b = [AdapterPool(sum(ranks) + 16, H, 1, b.dtype, dev, 1) for _ in range(layers)]
    for pools in (pools_a, pools_b):
        for pool in pools:
            for a in range(n_ad):
                pool.load_adapter(f"a{a}", ranks[a], workloads.ALPHA / ranks[a], [[None]])
            pool.buffer[0].copy_((torch.randn(pool.buffer[0].shape, generator=g, device=dev) * 0.02).to(b.dtype))
    x = [torch.randn(T, H, generator=g, device=dev).to(b.dtype) for _ in range(layers)]
    y = [torch.randn(T, H, generator=g, device=dev).to(b.dtype) for _ in range(layers)]
    v = [torch.zeros(T, max_r, dtype=b.dtype, device=dev) for _ in range(layers)]
    idx = torch.from_numpy(b.tok_adapter.astype(np.int64)).to(dev)
    packer = ops.Packer(T, n_ad, dev)
    pk = packer.pack(idx, pools_a[0].a_len, sort=False)
    P = pk.host_counts()["P"]
    tables = (pk.seg_len, pk.seg_rank, pk.seg_adapter, pk.seg_start)
    scales = pools_a[0].a_scaling

    def wview(pool):
        return pool.buffer[0].view(pool.buffer[0].shape[0], 32, H // 32)

    wa = [wview(p) for p in pools_a]
    wb = [wview(p) for p in pools_b]

    def shrink(l):
        p = pools_a[l]
        ops.atmm(v[l], x[l], wa[l], p.a_start, p.a_len, p.a_loc, idx, 0, scales, *tables, None, P)

    def expand(l):
        p = pools_b[l]
        ops.atmm(y[l], v[l], wb[l], p.a_start, p.a_len, p.a_loc, idx, 0, scales, *tables, None, P, apply_scale=True)

    e = 2
    rt = int(b.ranks[b.touched()].sum())
    lr = int(sum(int(l) * ranks[int(a)] for l, a in zip(b.req_len, b.req_adapter)))
    bytes_shrink = (T * H + rt * H) * e + lr * e
    bytes_expand = (2 * T * H + rt * H) * e + lr * e
    ms_s = _time_walk(shrink, layers, reps, warmup, eager)
    ms_e = _time_walk(expand, layers, reps, warmup, eager)
    ms_b = _time_walk(lambda l: (shrink(l), expand(l)), layers, reps, warmup, eager)
    if ops.device_status() != 0:
        raise SystemExit("a bounded wait gave up inside a kernel")
    peak, src = _peak()

    def gbs(nbytes, ms):
        return nbytes * layers / (ms * 1e-3) / 1e9

    flops = 4 * H * lr
    return {
        "bench": "ragged_atmm_dropin", "workload": b.name, "dtype": "fp16", "tokens": T, "segments": int(P),
        "adapters": n_ad, "ranks": ranks, "hidden": H, "layers_walked": layers,
        "shrink": {"us_per_call": ms_s * 1e3 / layers, "gbs": gbs(bytes_shrink, ms_s),
                   "frac": gbs(bytes_shrink, ms_s) / peak, "algorithmic_bytes": bytes_shrink},
        "expand": {"us_per_call": ms_e * 1e3 / layers, "gbs": gbs(bytes_expand, ms_e),
                   "frac": gbs(bytes_expand, ms_e) / peak, "algorithmic_bytes": bytes_expand},
        "both": {"us_per_pair": ms_b * 1e3 / layers, "gbs": gbs(bytes_shrink + bytes_expand, ms_b),
                 "frac": gbs(bytes_shrink + bytes_expand, ms_b) / peak,
                 "tokens_per_s": T * layers / (ms_b * 1e-3), "tflops": flops * layers / (ms_b * 1e-3) / 1e12},
        "peak_gbs": peak, "peak_source": src, "launch": "call by call" if eager else "one CUDA graph per walk, replayed",
    }


def bench_step(config: int, layers: int, reps: int, warmup: int, dev, shared_x: bool = False, gather_rows: int = 0,
               model: bool = False, graph: bool = False, ranks=None, split_rank_classes: bool = True):
    """A config through LoraStepEngine.step (device packer + one shrink and one
    expand launch): `layers` copies of the config's projections, every copy with its
    own pools and activations, CUDA events around each stage.  shared_x: q/k/v and
    up/gate of a copy read one X each (configs with the seven projections).
    model: the config's batch over the seven Qwen-VL-7B-shaped projections of every
    layer instead of the config's own single projection (a decode step of the whole
    model for config 1).  graph: the step is also captured into a CUDA graph and the
    replays are timed (`graph_ms_per_step`): what a serving loop that replays its
    decode step pays, without the host's launch path between the kernels.
    ranks: every adapter's rank redrawn from this list (seed 7) - the same batch with
    other ranks, e.g. [16] for the by-rank tables.  split_rank_classes=False: one launch per
    kernel even with adapters on both sides of rank 64."""
    from .engine import LoraStepEngine
    b = workloads.CONFIGS[config]()
    if ranks:
        b.ranks = np.random.default_rng(7).choice(np.array(ranks), size=b.n_adapters).astype(np.int64)
        b.name += "_ranks_" + "_".join(str(r) for r in ranks)
    if model:
        b.projections = list(workloads.PROJECTIONS)
        b.name += "_7proj"
    b.layers = layers
    input_of = None
    if shared_x:
        if len(b.projections) != len(workloads.SHARED_INPUT_OF):
            raise SystemExit("--shared-x needs a config with the seven projections (2 or 3)")
        input_of = list(workloads.SHARED_INPUT_OF)
    eng = LoraStepEngine(b.projections, b.ranks, b.scalings(), b.dtype, dev, layers, b.T, input_of=input_of,
                         split_rank_classes=split_rank_classes,
                         gather_rows_per_tile=gather_rows or None)
    eng.randomize_weights(seed=b.seed)
    g = torch.Generator(device=dev)
    g.manual_seed(b.seed + 7919)          # another stream than the weights'
    for l in range(layers):
        for p in range(len(b.projections)):
            if eng.input_of[p] == p:
                eng.x[l][p].normal_(generator=g)
            eng.y[l][p].normal_(generator=g)
    tok = torch.from_numpy(b.tok_adapter.astype(np.int64)).to(dev)
    for _ in range(warmup):
        packed = eng.step(tok)
    torch.cuda.synchronize()
    counts = packed.host_counts()
    names = ["pack"] + [n for n, _ in eng.phases()]
    ms = {n: [] for n in names}
    # Two timings per repetition, interleaved so that both see the same clocks.  (1) stage by
    # stage: one call per stage with events between them.  (2) the step itself: one call, nothing
    # recorded between its launches - a step that runs its kernels once per rank class overlaps
    # the two classes, which the per-stage calls cannot.
    tot, whole = [], []
    for _ in range(reps):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
        eng.step_timed(tok, ev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step(tok)
        e1.record()
        torch.cuda.synchronize()
        for i, n in enumerate(names):
            ms[n].append(ev[i].elapsed_time(ev[i + 1]))
        tot.append(ev[0].elapsed_time(ev[-1]))
        whole.append(e0.elapsed_time(e1))
    if ops.device_status() != 0:
        raise SystemExit("a bounded wait gave up inside a kernel")
    peak, src = _peak()
    step_ms = float(np.median(whole))
    nbytes, flops = b.algorithmic_bytes(input_of), b.algorithmic_flops()
    graph_ms = None
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            eng.step(tok)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g_ = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_):
            eng.step(tok)
        g_.replay()
        torch.cuda.synchronize()
        gt = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g_.replay()
            e1.record()
            torch.cuda.synchronize()
            gt.append(e0.elapsed_time(e1))
        graph_ms = float(np.median(gt))
        if ops.device_status() != 0:
            raise SystemExit("a bounded wait gave up inside a kernel")
    extra = {} if graph_ms is None else {"graph_ms_per_step": graph_ms,
                                         "graph_gbs": nbytes / (graph_ms * 1e-3) / 1e9,
                                         "graph_frac": nbytes / (graph_ms * 1e-3) / 1e9 / peak}
    return {**extra,
        "bench": "lora_step", "shared_x": bool(shared_x), "workload": b.name, "dtype": str(b.dtype).replace("torch.", ""), "tokens": b.T,
        "adapters": b.n_adapters, "adapters_touched": int(len(b.touched())),
        "ranks": sorted(set(int(r) for r in b.ranks)), "projections": len(b.projections), "layers": layers,
        "mma_tiles": counts["n_mma"], "gather_tiles": counts["n_gather"],
        "ms_per_step": step_ms, "phase_ms": {n: float(np.median(v)) for n, v in ms.items()},
        "phase_by_phase_ms": float(np.median(tot)),
        "tokens_per_s": b.T / (step_ms * 1e-3), "algorithmic_bytes": nbytes,
        "gbs": nbytes / (step_ms * 1e-3) / 1e9, "frac": nbytes / (step_ms * 1e-3) / 1e9 / peak,
        "tflops": flops / (step_ms * 1e-3) / 1e12, "peak_gbs": peak, "peak_source": src,
    }


def bench_fused(reps: int, warmup: int, dev, copies: int = 4, eager: bool = False):
    """The base projection with the expand folded in (vlr_fused_proj) on the prefill batch of
    config 2, one 4096 -> 4096 projection, bf16: shrink with the scale applied + the fused
    kernel, against the unfused sequence torch.mm + shrink + expand on the same tensors.
    `copies` independent sets of activations are walked per measurement (the base weight
    and the pools are shared: they are what a layer re-reads)."""
    b = workloads.config2()
    dtype = torch.bfloat16
    H, T, n_ad = workloads.H, b.T, b.n_adapters
    ranks = [int(r) for r in b.ranks]
    g = torch.Generator(device=dev)
    g.manual_seed(2)
    pa = AdapterPool(sum(ranks) + 16, H, 1, dtype, dev, 1)
    pb = AdapterPool(sum(ranks) + 16, H, 1, dtype, dev, 1)
    for pool in (pa, pb):
        for a in range(n_ad):
            pool.load_adapter(f"a{a}", ranks[a], workloads.ALPHA / ranks[a], [[None]])
        pool.buffer[0].copy_((torch.randn(pool.buffer[0].shape, generator=g, device=dev) * 0.02).to(dtype))
    W = (torch.randn(H, H, generator=g, device=dev) * 0.02).to(dtype)
    x = [torch.randn(T, H, generator=g, device=dev).to(dtype) for _ in range(copies)]
    y = [torch.empty(T, H, dtype=dtype, device=dev) for _ in range(copies)]
    v = [torch.zeros(T, 128, dtype=dtype, device=dev) for _ in range(copies)]
    idx = torch.from_numpy(b.tok_adapter.astype(np.int64)).to(dev)
    packer = ops.Packer(T, n_ad, dev)
    pk0 = packer.pack(idx, pa.a_len, sort=False)
    P = pk0.host_counts()["P"]
    tables = tuple(t.clone() for t in (pk0.seg_len, pk0.seg_rank, pk0.seg_adapter, pk0.seg_start))
    pk = packer.pack(idx, pa.a_len, sort=True)
    wa = pa.buffer[0].view(pa.buffer[0].shape[0], 32, H // 32)
    wb = pb.buffer[0].view(pb.buffer[0].shape[0], 32, H // 32)
    sc = pa.a_scaling

    def shrink(l, scaled):
        ops.atmm(v[l], x[l], wa, pa.a_start, pa.a_len, pa.a_loc, idx, 0, sc, *tables, None, P, apply_scale=scaled)

    def fused(l):
        ops.fused_proj(y[l], x[l], W, v[l], pb.buffer[0], pb.a_start, pb.a_loc, 0, pk)

    def unfused(l):
        torch.mm(x[l], W, out=y[l])
        shrink(l, False)
        ops.atmm(y[l], v[l], wb, pb.a_start, pb.a_len, pb.a_loc, idx, 0, sc, *tables, None, P, apply_scale=True)

    ms_f = _time_walk(fused, copies, reps, warmup, eager) / copies
    ms_sf = _time_walk(lambda l: (shrink(l, True), fused(l)), copies, reps, warmup, eager) / copies
    ms_mm = _time_walk(lambda l: torch.mm(x[l], W, out=y[l]), copies, reps, warmup, eager) / copies
    ms_u = _time_walk(unfused, copies, reps, warmup, eager) / copies
    if ops.device_status() != 0:
        raise SystemExit("a kernel reported a status")
    lr = int(b.ranks[b.tok_adapter].astype(np.int64).sum())
    flops_base, flops_exp = 2.0 * T * H * H, 2.0 * lr * H
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            m = json.load(f)
            peaks = {"bf16_tflops_burst": m.get("bf16_tflops"), "bf16_tflops_sustained": m.get("bf16_tflops_sustained")}
    except Exception:
        peaks = {"bf16_tflops_burst": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    tf = (flops_base + flops_exp) / (ms_f * 1e-3) / 1e12
    return {
        "bench": "fused_base_projection", "workload": b.name + " (q projection, bf16)", "tokens": T, "hidden": H,
        "ranks": sorted(set(ranks)), "mma_tiles": pk.host_counts()["n_mma"], "copies_walked": copies,
        "fused_kernel_ms": ms_f, "fused_kernel_tflops": tf,
        "frac_of_sustained_peak": tf / peaks["bf16_tflops_sustained"] if peaks.get("bf16_tflops_sustained") else None,
        "shrink_plus_fused_ms": ms_sf, "unfused_mm_shrink_expand_ms": ms_u, "torch_mm_alone_ms": ms_mm,
        "torch_mm_tflops": flops_base / (ms_mm * 1e-3) / 1e12,
        "hbm_bytes_fused": (2 * T * H + H * H) * 2, "hbm_bytes_unfused": (2 * T * H + H * H + 3 * T * H) * 2,
        "peaks": peaks,
    }


def trace_step(config: int, layers: int, phase: str, dev):
    """Stage timing of CTA 0 of one shrink or expand launch (clock64 stamps the kernels
    write while a trace buffer is set): medians over the stages of issue -> operands seen
    by the MMA thread -> epilogue / MMAs issued -> stage handed back, in cycles."""
    import ctypes
    from . import _lib
    from .engine import LoraStepEngine
    lib = _lib.load()
    if not hasattr(lib, "vlr_debug_set_trace"):
        raise SystemExit("the stage trace is compiled into debugging builds only: "
                         "python -m valora_b200.build --trace, then run with VLR_TRACE=1")
    b = workloads.CONFIGS[config]()
    b.layers = layers
    eng = LoraStepEngine(b.projections, b.ranks, b.scalings(), b.dtype, dev, layers, b.T)
    eng.randomize_weights(seed=b.seed)
    for l in range(layers):
        for p in range(len(b.projections)):
            eng.x[l][p].normal_()
            eng.y[l][p].normal_()
    tok = torch.from_numpy(b.tok_adapter.astype(np.int64)).to(dev)
    for _ in range(3):
        packed = eng.step(tok)
    torch.cuda.synchronize()
    cap = 1 << 16
    buf = torch.zeros(cap * 8, dtype=torch.int64, device=dev)
    bit = ops.PHASE_SHRINK_MMA if phase == "shrink" else ops.PHASE_EXPAND_MMA
    lib.vlr_debug_set_trace(ctypes.c_void_p(buf.data_ptr()), cap * 8)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    eng.plan.run(packed, eng.scales, 0, 0, phase_mask=bit | eng._gather_flag(), max_rank=max(eng.ranks))
    e1.record()
    torch.cuda.synchronize()
    lib.vlr_debug_set_trace(ctypes.c_void_p(0), 0)
    t = buf.cpu().numpy().reshape(cap, 8)
    n = int((t[:, 0] > 0).sum())
    t = t[:n]

    def med(a, c):
        return int(np.median(t[1:, a] - t[1:, c])) if n > 1 else 0

    out = {"bench": "stage_trace", "workload": b.name, "layers": layers, "phase": phase,
           "kernel_us": e0.elapsed_time(e1) * 1e3, "stages_of_cta0": n,
           "cycles_per_stage": float(t[:, 0].max() - t[:, 0].min()) / max(n - 1, 1),
           "issue_interval_median": int(np.median(np.diff(t[:, 0]))) if n > 1 else 0,
           "issue_to_operands_seen_median": med(1, 0)}
    if phase == "shrink":
        out["operands_seen_to_mmas_issued_median"] = med(2, 1)
        out["copies_issued_median"] = med(3, 0)
    else:
        out["operands_seen_to_epilogue_start_median"] = med(2, 1)
        out["epilogue_median"] = med(3, 2)
        out["issue_to_handed_back_median"] = med(3, 0)
        g = t[1:][t[1:, 4] > 0]                          # stages of gather tiles stamp their epilogue's phases
        if len(g):
            out["gather_stages"] = int(len(g))
            out["gather_epilogue_first_chunk_read_median"] = int(np.median(g[:, 4] - g[:, 2]))
            out["gather_epilogue_combine_median"] = int(np.median(g[:, 5] - g[:, 4]))
            out["gather_epilogue_store_median"] = int(np.median(g[:, 3] - g[:, 5]))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=1, choices=[0, 1, 2, 3, 4])
    ap.add_argument("--layers", type=int, default=0, help="independent copies walked (default: 32 / 4 / 32 / 8)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--eager", action="store_true", help="launch call by call (no CUDA graph), for profilers")
    ap.add_argument("--api", default="auto", choices=["auto", "dropin", "step"],
                    help="config 1 only: the 9-argument decode call (default) or the step API")
    ap.add_argument("--shared-x", action="store_true",
                    help="step API, configs 2 and 3: q/k/v and up/gate read one X per copy")
    ap.add_argument("--fused", action="store_true",
                    help="the base projection with the expand folded in, on config 2's q projection")
    ap.add_argument("--gather-rows", type=int, default=0, help="step API: rows per gather tile (default: the table's)")
    ap.add_argument("--model", action="store_true",
                    help="step API: the batch over the seven model projections per layer instead of the config's own")
    ap.add_argument("--graph", action="store_true", help="step API: also time replays of the step from a CUDA graph")
    ap.add_argument("--ranks", default="", help="step API: redraw every adapter's rank from this comma list (e.g. 16)")
    ap.add_argument("--no-rank-split", action="store_true",
                    help="step API: one launch per kernel even with adapters on both sides of rank 64")
    ap.add_argument("--trace", choices=["shrink", "expand"],
                    help="step API: print the stage timing of CTA 0 of one launch instead of timing steps")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device (there is no CPU fallback)")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.fused:
        print(json.dumps(bench_fused(args.reps, args.warmup, dev, eager=args.eager)))
    elif args.trace:
        default_layers = {0: 1, 1: 4, 2: 2, 3: 4, 4: 2}[args.config]
        print(json.dumps(trace_step(args.config, args.layers or default_layers, args.trace, dev)))
    elif args.config == 0:
        print(json.dumps(bench_atmm(args.layers or 32, args.reps, args.warmup, dev, args.eager)))
    elif args.config == 1 and args.api != "step":
        print(json.dumps(bench_bgmv(args.layers or 32, args.reps, args.warmup, dev, args.eager)))
    else:
        default_layers = {1: 32, 2: 4, 3: 32, 4: 8}[args.config]
        print(json.dumps(bench_step(args.config, args.layers or default_layers, args.reps, args.warmup, dev,
                                    args.shared_x, args.gather_rows, args.model, args.graph,
                                    [int(r) for r in args.ranks.split(",") if r], not args.no_rank_split)))


if __name__ == "__main__":
    main()
