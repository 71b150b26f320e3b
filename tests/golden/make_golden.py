#!/usr/bin/env python
"""Generate tests/golden/*.npz by RUNNING THE REFERENCE'S OWN PYTHON on CPU.

Run from the repository root in a container that has the reference checked out:

    python tests/golden/make_golden.py --reference /path/to/reference

Three pieces of the reference run unmodified here:

* ``ref_torch_groupgemm`` (test/kernel/vllm_utils.py:100-124).  The module's one
  third-party import (``vllm.lora.lora``, gone from current vllm) is satisfied
  by an empty stub so the file imports; the function body runs as shipped.
* ``ModelRpcServer.set_sgmm_args`` (valora/server/router/model_infer/
  model_rpc.py:265-374).  The module cannot be imported (rpyc, CUDA tensors at
  import time), so the function's source is cut out of the file with ``ast`` and
  executed as-is; ``device="cuda"`` / ``.cuda()`` are redirected to the CPU.
* ``MemoryAllocator`` (valora/common/mem_allocator.py), imported by file path
  with the same CPU redirection.

The outputs are the golden vectors that pin the oracle; nothing here is used
at test time except the files it writes.
"""
from __future__ import annotations

import argparse
import ast
import contextlib
import hashlib
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@contextlib.contextmanager
def cuda_to_cpu():
    """Redirect device='cuda' factory calls and Tensor.cuda() to the CPU."""
    names = ["ones", "zeros", "empty", "arange", "tensor", "full"]
    saved = {n: getattr(torch, n) for n in names}
    saved_cuda = torch.Tensor.cuda

    def wrap(fn):
        def inner(*a, **k):
            if str(k.get("device", "")).startswith("cuda"):
                k["device"] = "cpu"
            return fn(*a, **k)
        return inner

    for n in names:
        setattr(torch, n, wrap(saved[n]))
    torch.Tensor.cuda = lambda self, *a, **k: self
    try:
        yield
    finally:
        for n in names:
            setattr(torch, n, saved[n])
        torch.Tensor.cuda = saved_cuda


def load_groupgemm(ref):
    for name in ("vllm", "vllm.lora", "vllm.lora.lora"):
        if name not in sys.modules:
            sys.modules[name] = types.ModuleType(name)
    stub = sys.modules["vllm.lora.lora"]
    stub.LoRALayerWeights = type("LoRALayerWeights", (), {})
    stub.PackedLoRALayerWeights = type("PackedLoRALayerWeights", (), {})
    spec = importlib.util.spec_from_file_location(
        "ref_vllm_utils", os.path.join(ref, "test/kernel/vllm_utils.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.ref_torch_groupgemm


def load_set_sgmm_args(ref):
    path = os.path.join(ref, "valora/server/router/model_infer/model_rpc.py")
    src = open(path).read()
    tree = ast.parse(src)
    fn = None
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "set_sgmm_args":
            fn = node
    assert fn is not None
    text = ast.get_source_segment(src, fn)
    import textwrap
    ns = {"torch": torch}
    exec(textwrap.dedent(text), ns)
    return ns["set_sgmm_args"]


def load_allocator(ref):
    spec = importlib.util.spec_from_file_location(
        "ref_mem_allocator", os.path.join(ref, "valora/common/mem_allocator.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.MemoryAllocator


def u16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def gen_groupgemm(ref_fn, out):
    """Small ragged case (the benchmark's config-0 segment pattern scaled down)
    plus a digest of the full config 0."""
    cases = {}
    for dtype, tag in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        g = torch.Generator().manual_seed(7)
        Hs, ranks = 256, [8, 16, 16, 32]
        seg_len = [5, 33, 1, 1, 17, 40]
        seg_ad = [0, 1, 2, 3, 1, 0]
        T, R = sum(seg_len), max(ranks)
        x = torch.randn(T, Hs, generator=g).to(dtype)
        y0 = torch.randn(T, Hs, generator=g).to(dtype)
        wa = torch.zeros(4, R, Hs, dtype=dtype)          # shrink weights [n, out=r, in=H]
        wb = torch.zeros(4, Hs, R, dtype=dtype)          # expand weights [n, out=H, in=r]
        for a, r in enumerate(ranks):
            wa[a, :r] = (torch.randn(r, Hs, generator=g) * 0.02).to(dtype)
            wb[a, :, :r] = (torch.randn(Hs, r, generator=g) * 0.02).to(dtype)
        v = torch.zeros(T, R, dtype=dtype)
        ref_fn(v, x, wa, torch.tensor(seg_ad), torch.tensor(seg_len), len(seg_len), 1.0, "shrink")
        y = y0.clone()
        ref_fn(y, v, wb, torch.tensor(seg_ad), torch.tensor(seg_len), len(seg_len), 0.5, "expand")
        cases.update({
            f"{tag}_x": u16(x), f"{tag}_y0": u16(y0), f"{tag}_wa": u16(wa), f"{tag}_wb": u16(wb),
            f"{tag}_v": u16(v), f"{tag}_y": u16(y),
        })
    cases["seg_len"] = np.asarray(seg_len, np.int64)
    cases["seg_ad"] = np.asarray(seg_ad, np.int64)
    cases["ranks"] = np.asarray(ranks, np.int64)
    cases["expand_scaling"] = np.asarray([0.5], np.float32)

    # full config 0 through the reference function: keep only digests
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from valora_b200 import workloads
    b = workloads.config0()
    fl = workloads.make_floats(b)
    R = int(b.ranks.max())
    hi, ho = b.projections[0][1], b.projections[0][2]
    wa = torch.zeros(b.n_adapters, R, hi, dtype=b.dtype)
    wb = torch.zeros(b.n_adapters, ho, R, dtype=b.dtype)
    for a in range(b.n_adapters):
        r = int(b.ranks[a])
        wa[a, :r] = fl["A"][0][a].T
        wb[a, :, :r] = fl["B"][0][a].T
    v = torch.zeros(b.T, R, dtype=b.dtype)
    ref_fn(v, fl["X"][0], wa, torch.tensor(b.req_adapter), torch.tensor(b.req_len),
           len(b.req_len), 1.0, "shrink")
    cases["cfg0_v_sha256"] = np.frombuffer(hashlib.sha256(u16(v).tobytes()).digest(), np.uint8)
    # y = y0 + s * v B with the per-adapter scale: the reference function takes one
    # scalar, so it is called once per distinct scale on that scale's segments.
    y = fl["Y0"][0].clone()
    start = 0
    for L, a in zip(b.req_len.tolist(), b.req_adapter.tolist()):
        ys = y[start:start + L]
        ref_fn(ys, v[start:start + L], wb, torch.tensor([a]), torch.tensor([L]), 1,
               float(workloads.ALPHA / b.ranks[a]), "expand")
        start += L
    cases["cfg0_y_sha256"] = np.frombuffer(hashlib.sha256(u16(y).tobytes()).digest(), np.uint8)
    cases["cfg0_y_head"] = u16(y[:4, :64])
    np.savez_compressed(os.path.join(out, "groupgemm.npz"), **cases)


class _Batch:
    def __init__(self, adapter_dirs, input_lengths):
        self.adapter_dirs = list(adapter_dirs)
        self.input_lengths = list(input_lengths)
        self.requests = list(range(len(adapter_dirs)))
        self.num_problems = None


class _Self:
    class _IA:
        def __init__(self, dirs):
            self.adapter_dirs = dirs
    def __init__(self, dirs):
        self.infer_adapter = _Self._IA(dirs)


PACK_CASES = [
    # (adapter per request, input lengths, merged adapter or None)
    (["a"], [17], None),
    (["a", "a", "b"], [5, 7, 3], None),
    (["a", "b", "a", "a", "c"], [300, 12, 1, 44, 128], None),
    (["m", "m", "b", "c", "c"], [10, 20, 30, 40, 50], "m"),
    (["b", "m", "m", "c"], [9, 8, 7, 6], "m"),
    (["a", "b", "c", "d", "e", "f", "g", "h"], [256 + i for i in range(8)], None),
    (["x"] * 12, [3] * 12, None),
    (["x"] * 4 + ["y"] * 3 + ["x"] * 2, list(range(1, 10)), "y"),
]


def gen_pack(fn, out):
    res = {}
    with cuda_to_cpu():
        for ci, (dirs, lens, merged) in enumerate(PACK_CASES):
            for is_prefill in (True, False):
                b = _Batch(dirs, lens)
                srv = _Self(sorted(set(dirs)))
                r = fn(srv, b, is_prefill, merged)
                assert r is not None, (ci, is_prefill)
                oc, li, si = r
                tag = f"c{ci}_{'p' if is_prefill else 'd'}"
                res[tag + "_output_counts"] = oc.numpy().astype(np.int64)
                res[tag + "_lora_ids"] = li.numpy().astype(np.int64)
                res[tag + "_start_ids"] = si.numpy().astype(np.int64)
                np_ = b.num_problems
                res[tag + "_num_problems"] = np.asarray([np_[0], np_[1][0], np_[1][1]], np.int64)
    np.savez_compressed(os.path.join(out, "set_sgmm_args.npz"), **res)


def gen_alloc(MemoryAllocator, out):
    res = {}
    with cuda_to_cpu():
        m = MemoryAllocator(tot_size=64, cache_size=16, dtype=torch.float16, head_num=2,
                            head_dim=4, layer_num=1)
        a = m.alloc(10)
        b = m.alloc(7)
        m.free(a[2:6])
        c = m.alloc(9)
        m.free(b)
        d = m.alloc(12)
        res = dict(a=a.numpy(), b=b.numpy(), c=c.numpy(), d=d.numpy(),
                   state=m.mem_state.numpy().astype(np.uint8),
                   can_use=np.asarray([m.can_use_mem_size], np.int64))
        try:
            m.alloc(1000)
            res["raised"] = np.asarray([0])
        except Exception:
            res["raised"] = np.asarray([1])
    np.savez_compressed(os.path.join(out, "mem_allocator.npz"), **res)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    torch.set_num_threads(1)  # fixed reduction order for the digests
    gen_groupgemm(load_groupgemm(args.reference), args.out)
    gen_pack(load_set_sgmm_args(args.reference), args.out)
    gen_alloc(load_allocator(args.reference), args.out)
    print("golden vectors written to", args.out)


if __name__ == "__main__":
    main()
