#!/usr/bin/env python
"""Benchmark of the multi-LoRA batching step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the continuous mixed batch (8 prefill requests + 384 decode tokens,
64 adapters of rank 64, adapter skew 0.8) over 32 layers x 7 Qwen-VL-7B-shaped
projections in bf16; the batch is packed on the device every step.  A step is
one pass of pack + shrink + expand over all 224 (layer, projection) problems.
Prints ONE JSON line.  With N > 1 (under torchrun) every rank runs its own
batch over its own adapter group (weak scaling, no data-path collective).

--impl reference times the reference's CPU torch path (the per-segment
mm(mm(x, A), B) * s walk, restated in oracle/) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from valora_b200 import shard, workloads  # noqa: E402

METRIC = "lora_tokens_per_s"
UNIT = "tokens/s"
LAYERS = 32


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def make_batch(rank: int):
    """Config 3 for rank 0 (seed 3); other ranks draw their own batch of the same
    composition from seed 3 + 1000 * rank over their own 64 adapters."""
    b = workloads.config3(layers=LAYERS)
    if rank == 0:
        return b
    rng = np.random.default_rng(3 + 1000 * rank)
    pre_len = 256 + workloads._text_lengths(rng, 8)
    req_ad = rng.choice(64, size=8 + 384, p=workloads.zipf_probs(64, 0.8)).astype(np.int32)
    req_len = np.concatenate([pre_len, np.ones(384, np.int64)])
    b.tok_adapter = workloads._tok_from_requests(req_ad, req_len)
    b.req_adapter, b.req_len, b.seed = req_ad, req_len, 3 + 1000 * rank
    return b


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                mhz, mx = float(f[1]), float(f[2])
            except ValueError:
                continue
            smax = mx
            if t0 - 0.05 <= ts <= t1 + 0.15:
                sm.append(mhz)
                for n, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        if not sm:
            sm = [float(x[1].split(",")[1]) for x in self.lines[-3:] if len(x[1].split(",")) > 2] or [0.0]
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy kernel)"
    except Exception:
        return 6650.0, "fallback (earlier measurement on this pool)"


def phase_bytes(batch, tiles, n_mma, n_gather, merged):
    """Algorithmic HBM bytes of each kernel launch of one step: the rows a kernel
    covers (X once for a shrink; Y0 read + Y write for an expand) plus the weights
    of every adapter it touches, once.  2-byte elements; V and metadata excluded.
    merged: one shrink and one expand launch cover both kinds of tile."""
    mma, gat = tiles[:n_mma], tiles[n_mma:n_mma + n_gather]
    rows = {"mma": int(mma[:, 4].sum()) if n_mma else 0, "gather": int(gat[:, 4].sum()) if n_gather else 0}
    ads = {"mma": np.unique(mma[:, 1]) if n_mma else np.zeros(0, np.int64),
           "gather": np.unique(gat[:, 1]) if n_gather else np.zeros(0, np.int64)}
    out = {}

    def add(name_s, name_e, nrows, adapters):
        rk = int(batch.ranks[adapters].sum()) if len(adapters) else 0
        out[name_s] = sum(nrows * hi + rk * hi for _, hi, _ in batch.projections) * 2 * batch.layers
        out[name_e] = sum(2 * nrows * ho + rk * ho for _, _, ho in batch.projections) * 2 * batch.layers

    if merged:
        add("shrink", "expand", rows["mma"] + rows["gather"], np.union1d(ads["mma"], ads["gather"]).astype(np.int64))
    else:
        for kind in ("mma", "gather"):
            add("shrink_" + kind, "expand_" + kind, rows[kind], ads[kind].astype(np.int64))
    return out, rows


def cpu_baseline_layer(batch, reps=2, threads=None):
    """The reference's torch path on the host: one layer (7 projections) of the
    batch, in the batch dtype, walking the adapter-sorted segments."""
    import oracle
    if threads:
        torch.set_num_threads(threads)
    pk = oracle.pack_sorted_ref(batch.tok_adapter, batch.ranks)
    g = torch.Generator().manual_seed(batch.seed)
    sc = batch.scalings()
    data = []
    for _, hi, ho in batch.projections:
        A = [(torch.randn(hi, int(r), generator=g) * 0.02).to(batch.dtype) for r in batch.ranks]
        B = [(torch.randn(int(r), ho, generator=g) * 0.02).to(batch.dtype) for r in batch.ranks]
        x = torch.randn(batch.T, hi, generator=g).to(batch.dtype)
        y0 = torch.randn(batch.T, ho, generator=g).to(batch.dtype)
        data.append((y0, x, A, B))
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        for y0, x, A, B in data:
            oracle.ragged_lora_ref(y0, x, A, B, pk["seg_len"], pk["seg_adapter"], sc)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def run_reference(args, rank, world):
    if rank != 0:
        return
    batch = make_batch(0)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    for _ in range(max(args.warmup, 1) and 1):
        cpu_baseline_layer(batch, reps=1)
    times = [cpu_baseline_layer(batch, reps=1) for _ in range(max(1, min(args.steps, 3)))]
    t_layer = float(np.mean(times))
    t_step = t_layer * LAYERS
    v = batch.T / t_step
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": 1, "ms_per_step": t_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": batch.name, "tokens": batch.T, "layers": LAYERS,
                   "projections": len(batch.projections), "adapters": batch.n_adapters, "rank": 64},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "1 of 32 layers (7 projections, whole batch) per step, time x 32"},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


_JSON_FD = None


def emit(line):
    """Write the result line to the process's original stdout."""
    sys.stdout.flush()
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        os.write(1, data)
    else:
        os.write(_JSON_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=LAYERS, help="for profiling small cases only")
    ap.add_argument("--gather-path", default="mma", choices=["mma", "simt"],
                    help="decode rows on the tensor-core kernels (gathered rows) or on the SIMT gather kernels")
    args = ap.parse_args()

    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    # stdout carries the one JSON line and nothing else: whatever a library writes there while the
    # bench runs (NCCL prints its version line to stdout) goes to stderr instead
    sys.stdout.flush()
    global _JSON_FD
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from valora_b200.engine import LoraStepEngine
    from valora_b200 import ops

    batch = make_batch(rank)
    batch.layers = args.layers
    T = batch.T
    warmup = max(args.warmup, 3)
    eng = LoraStepEngine(batch.projections, batch.ranks, batch.scalings(), batch.dtype, dev,
                         args.layers, T, gather_path=args.gather_path)
    eng.randomize_weights(seed=batch.seed)
    g = torch.Generator(device=dev)
    g.manual_seed(batch.seed)
    for layer in range(args.layers):
        for p in range(len(batch.projections)):
            eng.x[layer][p].normal_(generator=g)
            eng.y[layer][p].normal_(generator=g)
    tok = torch.from_numpy(batch.tok_adapter.astype(np.int64)).to(dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (untimed)
    for _ in range(warmup):
        packed = eng.step(tok)
    torch.cuda.synchronize()
    if ops.device_status() != 0:
        raise SystemExit("a bounded wait gave up inside a kernel during warm-up")
    counts = packed.host_counts()
    tiles_h = packed.tiles.cpu().numpy()
    pbytes, rows = phase_bytes(batch, tiles_h, counts["n_mma"], counts["n_gather"],
                               merged=args.gather_path == "mma")
    kernel_names = [n for n, _ in eng.phases()]
    n_ev = 2 + len(kernel_names)

    # ---- timed region: K steps, events between the stages of every step
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(n_ev)] for _ in range(K)]
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.25)
    barrier()
    t0 = time.time()
    for k in range(K):
        eng.step_timed(tok, ev[k])
    torch.cuda.synchronize()
    t1 = time.time()
    barrier()
    clocks = sampler.stop(t0, t1)
    total_ms = ev[0][0].elapsed_time(ev[K - 1][n_ev - 1])
    names = ["pack"] + kernel_names
    phase_ms = {n: float(np.mean([ev[k][i].elapsed_time(ev[k][i + 1]) for k in range(K)]))
                for i, n in enumerate(names)}
    if ops.device_status() != 0:
        raise SystemExit("a bounded wait gave up inside a kernel during the timed region")

    # max over ranks of the device time, sum over ranks of the tokens served
    ms_per_step, tokens = shard.reduce_timing(total_ms / K, float(T), device=dev)
    value = tokens / (ms_per_step * 1e-3)

    # ---- end to end: pinned host buffers in, Y back out, every step
    e2e = None
    if args.e2e_steps > 0:
        xh = [torch.empty((T, hi), dtype=batch.dtype).pin_memory() for _, hi, _ in batch.projections]
        yh = [torch.empty((T, ho), dtype=batch.dtype).pin_memory() for _, _, ho in batch.projections]
        oh = [torch.empty((T, ho), dtype=batch.dtype).pin_memory() for _, _, ho in batch.projections]
        for t in xh + yh:
            t.normal_()
        tok_h = torch.from_numpy(batch.tok_adapter.astype(np.int64)).pin_memory()
        tok_d = torch.empty(T, dtype=torch.int64, device=dev)
        x_all, y_all, o_all = [xh] * args.layers, [yh] * args.layers, [oh] * args.layers
        eng.step_host(tok_h, x_all, y_all, tok_d, y_out_host=o_all)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            h2d, d2h = eng.step_host(tok_h, x_all, y_all, tok_d, y_out_host=o_all)
        e1.record()
        torch.cuda.synchronize()
        barrier()
        ems, _ = shard.reduce_timing(e0.elapsed_time(e1) / args.e2e_steps, 0.0, device=dev)
        e2e = {"value": tokens / (ems * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": ems,
               "note": "H2D, kernels and D2H pipelined by layer over three streams; one layer's pinned "
                       "source buffers (read-only) and one layer's pinned sink buffers stand for all layers"}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    dom = max(kernel_names, key=lambda n: phase_ms[n])
    achieved = pbytes[dom] / (phase_ms[dom] * 1e-3) / 1e9
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        try:
            traffic = json.load(open(tpath)).get(dom, {}).get("bytes_per_launch_full")
        except Exception:
            traffic = None
    step_bytes = batch.algorithmic_bytes()
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": batch.name, "tokens_per_gpu": T, "layers": args.layers,
                   "projections": len(batch.projections), "adapters_per_gpu": batch.n_adapters, "rank": 64,
                   "parallelism": f"adapter-group x{world}", "gather_path": args.gather_path, "mma_tiles": counts["n_mma"],
                   "gather_tiles": counts["n_gather"], "rows_mma": rows["mma"], "rows_gather": rows["gather"],
                   "l2": "inputs larger than L2 (every step streams tens of GB of distinct buffers)",
                   "algorithmic_bytes_per_step": step_bytes,
                   "step_gbs": step_bytes / (ms_per_step * 1e-3) / 1e9,
                   "step_frac_of_peak": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak,
                   "tflops": batch.algorithmic_flops() / (ms_per_step * 1e-3) / 1e12,
                   "phase_ms": phase_ms, "phase_algorithmic_bytes": pbytes},
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": (5 + len(kernel_names)) * K,
        "roofline": {"kernel": dom, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": pbytes[dom], "ms_per_launch": phase_ms[dom]},
    }
    if not args.no_cpu_baseline and world == 1:
        threads = os.cpu_count() or 1
        t_layer = cpu_baseline_layer(workloads.config3(layers=LAYERS), reps=2, threads=threads)
        line["cpu_baseline"] = {"value": T / (t_layer * LAYERS), "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": "1 of 32 layers (7 projections, whole batch), best of 2, time x 32"}
    else:
        line["cpu_baseline"] = None
    emit(line)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
