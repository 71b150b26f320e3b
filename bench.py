#!/usr/bin/env python
"""Benchmark of the multi-LoRA batching step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload: the continuous mixed batch (8 prefill requests + 384 decode
tokens, 64 adapters of rank 64, adapter skew 0.8) over 32 layers x 7
Qwen-VL-7B-shaped projections in bf16; the batch is packed on the device every
step.  A step is one call: the packer's launches, then one shrink and one
expand launch that cover all 224 (layer, projection) problems.  Before anything
is timed, one step on fresh buffers is compared with the CPU oracle on a sample
of the 224 problems (`parity` in the output; the run fails if it is off).
With N > 1 (under torchrun) every rank runs its own batch of that composition
over its own adapter group (weak scaling, no data-path collective).

Second block (`config4`): the box-scale batch - 16384 tokens over 1024 resident
adapters of ranks 16..128, generated once from seed 4 - partitioned over the N
GPUs by adapter group (adapter a lives on GPU a % N), once plainly and once
with the most popular adapters replicated on every GPU; per-rank and whole-box
figures.

Prints ONE JSON line.

--impl reference times the reference's CPU torch path (the per-segment
mm(mm(x, A), B) * s walk, restated in oracle/ and pinned bit-exactly to the
reference's own function by the committed golden vectors) on the host cores.
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
CFG4_LAYERS = 8          # independent copies of config 4's projection walked per step (larger than L2 together)
CFG4_TOPK = 16           # adapters replicated on every GPU in the second config-4 run
TOL = 1e-2
OWN_ALLOWANCE = 2e-3
ACT_SEED = 7919          # activations are drawn from another stream than the weights


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


def config_dict(batch, world, layers):
    """The workload's identity: the same keys and values in both arms."""
    return {"workload": batch.name, "tokens_per_gpu": batch.T, "layers": layers,
            "projections": len(batch.projections), "adapters_per_gpu": batch.n_adapters, "rank": 64,
            "parallelism": f"adapter-group x{world}",
            "l2": "inputs larger than L2 (every step streams tens of GB of distinct buffers)"}


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


# --------------------------------------------------------------------------- parity (the oracle as checker)
def out_tolerance(ref32, dtype):
    """1e-2; where the 16-bit output grid is too coarse for that (bf16, |y| >= 4): half an ulp
    of the output type plus 2e-3 for the kernels' own error (16-bit shrink result)."""
    prec = 8 if dtype == torch.bfloat16 else 11
    mag = ref32.abs().clamp_min(1e-30)
    half_ulp = torch.exp2(torch.floor(torch.log2(mag)) - prec)
    return torch.maximum(torch.full_like(ref32, TOL), half_ulp + OWN_ALLOWANCE), half_ulp


def parity_step(eng, tok_np, ranks, scalings, dtype, sample):
    """One step on the engine's current buffers, checked on the host against the fp32
    oracle for the (layer, projection) problems in `sample`.  Returns the parity record;
    max_excess <= 0 means every element is within its bound."""
    import oracle
    T = int(tok_np.shape[0])
    dev = eng.device
    y0 = {lp: eng.y[lp[0]][lp[1]][:T].cpu() for lp in sample}
    x = {lp: eng.x[lp[0]][lp[1]][:T].cpu() for lp in sample}
    packed = eng.step(torch.from_numpy(tok_np.astype(np.int64)).to(dev))
    torch.cuda.synchronize()
    pk = oracle.pack_sorted_ref(tok_np, ranks)
    perm = torch.from_numpy(pk["perm"].astype(np.int64))
    packing_ok = bool(np.array_equal(packed.perm[:T].cpu().numpy(), pk["perm"]))
    touched = np.unique(tok_np)
    worst, worst_own, worst_abs = -1.0, 0.0, 0.0
    for (l, p) in sample:
        A = [None] * len(ranks)
        B = [None] * len(ranks)
        for a in touched:
            Aa, Ba = eng.adapter_weights(l, p, int(a))
            A[int(a)], B[int(a)] = Aa.cpu(), Ba.cpu()
        ref = oracle.ragged_lora_ref_fp32(y0[(l, p)][perm], x[(l, p)][perm], A, B, pk["seg_len"],
                                          pk["seg_adapter"], scalings)
        got = eng.y[l][p][:T].cpu()[perm].float()
        err = (got - ref).abs()
        bound, half_ulp = out_tolerance(ref, dtype)
        worst = max(worst, float((err - bound).max()))
        worst_own = max(worst_own, float((err - half_ulp).clamp_min(0).max()))
        worst_abs = max(worst_abs, float(err.max()))
    return {"checked_problems": len(sample), "problems": [list(lp) for lp in sample],
            "oracle": "ragged_lora_ref_fp32 (fp32 arithmetic on the 16-bit inputs)",
            "bound": "1e-2, or half an ulp of bf16 + 2e-3 where that is larger (|y| >= 4)",
            "max_excess": worst, "max_abs_err": worst_abs, "max_err_beyond_half_ulp": worst_own,
            "packing_bit_exact": packing_ok, "ok": bool(worst <= 0.0 and packing_ok)}


# --------------------------------------------------------------------------- CPU legs
def cpu_layer_data(batch):
    g = torch.Generator().manual_seed(batch.seed)
    data = []
    for _, hi, ho in batch.projections:
        A = [(torch.randn(hi, int(r), generator=g) * 0.02).to(batch.dtype) for r in batch.ranks]
        B = [(torch.randn(int(r), ho, generator=g) * 0.02).to(batch.dtype) for r in batch.ranks]
        x = torch.randn(batch.T, hi, generator=g).to(batch.dtype)
        y0 = torch.randn(batch.T, ho, generator=g).to(batch.dtype)
        data.append((y0, x, A, B))
    return data


def cpu_walk(batch, data, pk, walks):
    """The reference's torch path on the host: `walks` passes over one layer's seven
    projections of the whole batch, in the batch dtype, segment by segment."""
    import oracle
    sc = batch.scalings()
    t0 = time.perf_counter()
    for _ in range(walks):
        for y0, x, A, B in data:
            oracle.ragged_lora_ref(y0, x, A, B, pk["seg_len"], pk["seg_adapter"], sc)
    return time.perf_counter() - t0


def run_reference(args, rank, world):
    """The reference arm: rank 0 alone, all host threads.  A step = the 32 layers of the
    headline batch, as 32 walks over one layer's tensors (the 32 layers differ only in
    their values; one layer's 0.8 GB already exceeds the host caches)."""
    if rank != 0:
        return
    import oracle
    batch = make_batch(0)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    data = cpu_layer_data(batch)
    pk = oracle.pack_sorted_ref(batch.tok_adapter, batch.ranks)
    t_probe = cpu_walk(batch, data, pk, 1)
    # bound the whole run to a few minutes: fewer walks per step if the host is slow
    total_steps = max(args.steps, 1) + max(args.warmup, 0)
    walks = LAYERS
    while walks > 1 and t_probe * walks * total_steps > 240.0:
        walks //= 2
    for _ in range(max(args.warmup, 0)):
        cpu_walk(batch, data, pk, walks)
    times = [cpu_walk(batch, data, pk, walks) * (LAYERS / walks) for _ in range(max(args.steps, 1))]
    t_step = float(np.mean(times))
    v = batch.T / t_step
    sample = (f"each step = {walks} walks over one layer's tensors (7 projections, whole batch)"
              + ("" if walks == LAYERS else f", time x {LAYERS // walks}"))
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": max(args.warmup, 0), "ms_per_step": t_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(batch, args.gpus, LAYERS),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
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


def gather_objects(dist, obj, world):
    if dist is None:
        return [obj]
    out = [None] * world
    dist.all_gather_object(out, obj)
    return out


# --------------------------------------------------------------------------- config 4, sharded by adapter group
def config4_block(dist, dev, rank, world, steps, warmup, peak):
    """The box-scale batch partitioned over the GPUs by adapter group.  Every rank
    regenerates the global batch from seed 4 and keeps what it owns (shard.route): its
    pools hold only its adapters (plus, in the second run, the replicated ones)."""
    from valora_b200.engine import LoraStepEngine
    from valora_b200 import ops
    g = workloads.config4()
    H = workloads.H
    counts = np.bincount(g.tok_adapter, minlength=g.n_adapters)
    out = {"workload": "cfg4_box_bf16", "tokens_per_step": g.T, "adapters_resident": g.n_adapters,
           "layers": CFG4_LAYERS, "hidden": H, "partition": "adapter a on GPU a % N, requests routed whole"}
    runs = [("partitioned", None)]
    if world > 1:
        runs.append(("replicated_top%d" % CFG4_TOPK, shard.pick_replicated(counts, CFG4_TOPK)))
    for name, hot in runs:
        if hot is None:
            s = shard.route(g.req_adapter, g.req_len, world, rank)
        else:
            s = shard.route_with_replication(g.req_adapter, g.req_len, world, rank, hot, g.n_adapters)
        ranks = shard.local_ranks(g.ranks, world, rank, hot)
        T = s.T
        rec = {"T": T, "ms": None}
        if T > 0:
            scal = (workloads.ALPHA / ranks).astype(np.float32)
            eng = LoraStepEngine([("q", H, H)], ranks, scal, torch.bfloat16, dev, CFG4_LAYERS, T)
            eng.randomize_weights(seed=4 + rank)
            gen = torch.Generator(device=dev)
            gen.manual_seed(4 + rank + ACT_SEED)
            for l in range(CFG4_LAYERS):
                eng.x[l][0].normal_(generator=gen)
                eng.y[l][0].normal_(generator=gen)
            tok_np = s.tok_adapter.astype(np.int64)
            par = parity_step(eng, tok_np, ranks, scal, torch.bfloat16, [(0, 0), (CFG4_LAYERS - 1, 0)])
            tok = torch.from_numpy(tok_np).to(dev)
            for _ in range(warmup):
                eng.step(tok)
            torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        if T > 0:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                eng.step(tok)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            touched = np.unique(tok_np)
            nbytes = (3 * T * H + 2 * int(ranks[touched].sum()) * H) * 2 * CFG4_LAYERS
            rec.update(ms=ms, gbs=nbytes / (ms * 1e-3) / 1e9, frac=nbytes / (ms * 1e-3) / 1e9 / peak,
                       algorithmic_bytes=nbytes, adapters_touched=int(len(touched)),
                       parity_max_excess=par["max_excess"], parity_ok=par["ok"],
                       status=int(ops.device_status()))
            del eng
            torch.cuda.empty_cache()
        if dist is not None:
            dist.barrier()
        per_rank = gather_objects(dist, rec, world)
        loads = [r["T"] for r in per_rank]
        ms_max = max((r["ms"] or 0.0) for r in per_rank)
        out[name] = {
            "per_rank": per_rank,
            "load_max_over_mean": max(loads) / (sum(loads) / len(loads)),
            "ms_per_step_max": ms_max,
            "box_tokens_per_s": sum(loads) / (ms_max * 1e-3) if ms_max > 0 else None,
            "parity_ok": all(r.get("parity_ok", True) for r in per_rank),
            "replicated_adapters": None if hot is None else [int(a) for a in hot],
        }
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-config4", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="for profiler runs only")
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
    g.manual_seed(batch.seed + ACT_SEED)
    for layer in range(args.layers):
        for p in range(len(batch.projections)):
            eng.x[layer][p].normal_(generator=g)
            eng.y[layer][p].normal_(generator=g)
    tok = torch.from_numpy(batch.tok_adapter.astype(np.int64)).to(dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- parity of the launch that is timed: one step on the fresh buffers against the fp32 oracle,
    # every projection shape, first / middle / last layer (on every rank: each has its own batch)
    parity = None
    if not args.no_parity:
        L = args.layers
        mid = L // 2
        sample = sorted(set([(0, 0), (0, 4), (0, 6), (mid, 1), (mid, 5), (mid, 6),
                             (L - 1, 2), (L - 1, 3), (L - 1, 4), (L - 1, 6)]))
        parity = parity_step(eng, batch.tok_adapter, batch.ranks, batch.scalings(), batch.dtype, sample)
        if ops.device_status() != 0:
            raise SystemExit("a bounded wait gave up inside a kernel during the parity step")
        if not parity["ok"]:
            emit({"metric": METRIC, "value": None, "parity": parity, "error": "parity check failed"})
            raise SystemExit(f"parity check failed on rank {rank}: {parity}")

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
    my_ms = total_ms / K
    ms_per_step, tokens = shard.reduce_timing(my_ms, float(T), device=dev)
    value = tokens / (ms_per_step * 1e-3)
    peak, peak_src = measured_peak()
    step_bytes = batch.algorithmic_bytes()

    # ---- end to end: pinned host buffers in, Y back out, every step.  q/k/v and up/gate read one
    # activation buffer each, as the reference's caller hands one input to the three projections, so
    # a shared X crosses the link once.  Same pools, same Y buffers as the resident engine.
    e2e = None
    e2e_rank = None
    if args.e2e_steps > 0:
        input_of = list(workloads.SHARED_INPUT_OF)
        eng2 = LoraStepEngine(batch.projections, batch.ranks, batch.scalings(), batch.dtype, dev,
                              args.layers, T, gather_path=args.gather_path, alloc_activations=False,
                              input_of=input_of, share_pools_with=eng)
        eng2.x = [[eng.x[l][input_of[p]] for p in range(len(batch.projections))] for l in range(args.layers)]
        eng2.y = eng.y
        eng2.build_plan()
        xh = [torch.empty((T, hi), dtype=batch.dtype).pin_memory() for _, hi, _ in batch.projections]
        yh = [torch.empty((T, ho), dtype=batch.dtype).pin_memory() for _, _, ho in batch.projections]
        oh = [torch.empty((T, ho), dtype=batch.dtype).pin_memory() for _, _, ho in batch.projections]
        for t in xh + yh:
            t.normal_()
        tok_h = torch.from_numpy(batch.tok_adapter.astype(np.int64)).pin_memory()
        tok_d = torch.empty(T, dtype=torch.int64, device=dev)
        x_all, y_all, o_all = [xh] * args.layers, [yh] * args.layers, [oh] * args.layers
        eng2.step_host(tok_h, x_all, y_all, tok_d, y_out_host=o_all)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            h2d, d2h = eng2.step_host(tok_h, x_all, y_all, tok_d, y_out_host=o_all)
        e1.record()
        torch.cuda.synchronize()
        barrier()
        my_ems = e0.elapsed_time(e1) / args.e2e_steps
        ems, _ = shard.reduce_timing(my_ems, 0.0, device=dev)
        e2e_rank = {"ms": my_ems, "h2d_gbs": h2d / (my_ems * 1e-3) / 1e9, "d2h_gbs": d2h / (my_ems * 1e-3) / 1e9}
        e2e = {"value": tokens / (ems * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": ems,
               "note": "H2D, kernels and D2H pipelined by layer over three streams; q/k/v and up/gate share "
                       "one X each (copied once); one layer's pinned source buffers (read-only) and one "
                       "layer's pinned sink buffers stand for all layers"}
        if ops.device_status() != 0:
            raise SystemExit("a bounded wait gave up inside a kernel during the end-to-end steps")
        del eng2, xh, yh, oh

    per_rank = gather_objects(dist, {
        "rank": rank, "T": T, "ms_per_step": my_ms, "phase_ms": phase_ms,
        "step_frac_of_peak": step_bytes / (my_ms * 1e-3) / 1e9 / peak,
        "parity_max_excess": None if parity is None else parity["max_excess"],
        "e2e": e2e_rank, "power_cap_seen": "sw_power_cap" in clocks.get("reasons", []),
        "sm_mhz": clocks.get("sm_mhz")}, world)

    # ---- config 4: one global batch partitioned by adapter group
    cfg4 = None
    if not args.no_config4 and args.layers == LAYERS:
        del eng
        torch.cuda.empty_cache()
        cfg4 = config4_block(dist, dev, rank, world, max(3, min(K, 10)), 3, peak)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    dom = max(kernel_names, key=lambda n: phase_ms[n])
    achieved = pbytes[dom] / (phase_ms[dom] * 1e-3) / 1e9
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        try:
            traffic = json.load(open(tpath)).get(dom, {}).get("bytes_per_launch_full")
        except Exception:
            traffic = None
    if e2e is not None and world > 1:
        e2e["aggregate_h2d_gbs"] = sum(r["e2e"]["h2d_gbs"] for r in per_rank)
        e2e["aggregate_d2h_gbs"] = sum(r["e2e"]["d2h_gbs"] for r in per_rank)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": config_dict(batch, world, args.layers),
        "detail": {"gather_path": args.gather_path, "mma_tiles": counts["n_mma"],
                   "gather_tiles": counts["n_gather"], "rows_mma": rows["mma"], "rows_gather": rows["gather"],
                   "algorithmic_bytes_per_step": step_bytes,
                   "step_gbs": step_bytes / (ms_per_step * 1e-3) / 1e9,
                   "step_frac_of_peak": step_bytes / (ms_per_step * 1e-3) / 1e9 / peak,
                   "tflops": batch.algorithmic_flops() / (ms_per_step * 1e-3) / 1e12,
                   "phase_ms": phase_ms, "phase_algorithmic_bytes": pbytes,
                   "launches_per_step": "packer (4 small kernels) + 1 memset + shrink + expand: one call, "
                                        "two launches that cover all problems",
                   "per_rank": per_rank},
        "parity": parity,
        "clocks": clocks,
        "e2e": e2e,
        "gpu_launches": (4 + len(kernel_names)) * K,
        "roofline": {"kernel": dom, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": pbytes[dom], "ms_per_launch": phase_ms[dom]},
        "config4": cfg4,
    }
    if not args.no_cpu_baseline and world == 1:
        import oracle
        threads = os.cpu_count() or 1
        torch.set_num_threads(threads)
        b0 = workloads.config3(layers=LAYERS)
        data = cpu_layer_data(b0)
        pk = oracle.pack_sorted_ref(b0.tok_adapter, b0.ranks)
        cpu_walk(b0, data, pk, 1)
        walks = 8
        t = min(cpu_walk(b0, data, pk, walks) for _ in range(2)) * (LAYERS / walks)
        line["cpu_baseline"] = {"value": T / t, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": f"{walks} walks over one layer's tensors (7 projections, whole batch), "
                                          f"best of 2, time x {LAYERS // walks}"}
    else:
        line["cpu_baseline"] = None
    emit(line)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
