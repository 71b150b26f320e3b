#!/usr/bin/env python
"""Generate tests/golden/caller_trace.{json,npz} by RUNNING THE REFERENCE'S OWN
CALLER CODE on CPU and recording every operator call it makes.

    python tests/golden/make_caller_trace.py --reference /path/to/reference

The callers of the two operator entry points are methods of
LoraUnorderedBatchInfer (valora/models/peft/lora_unordered_batch_infer.py):
_lora_get_qkv (:876-1071), _lora_get_o (:1563-1683), _batch_lora_get_qkv
(:562-874) and _batch_lora_get_o (:1453-1561).  The module cannot be imported
(rpyc, CUDA tensors at import time, triton kernels), so - as make_golden.py does
for set_sgmm_args - the methods' source is cut out of the file with ``ast`` and
executed unmodified, with

* ``self`` a plain namespace holding what the methods read (pool buffers, index
  tables, the problem table, the zeroed delta buffers, a base model made of
  random projection weights),
* ``dispatch_sgmm`` / ``dispatch_bgmv`` recorders that note how every argument is
  bound (which tensor, which view of it, which integers - the reference passes
  ``tb_z`` where the sixth tile integer belongs, slices ``[delora_tk_index:]``
  of activations and outputs, and reads ONE value_buffer as [H_out, r] through
  BGMV and as [r, H_out] through ATMM) and then carry the call out with the CPU
  oracle, so that the methods run to their end and return q / o,
* ``torch.cuda.synchronize`` a no-op and the rotary embedding (base-model work,
  not part of the operator) a no-op.

What is written: the tensors the calls touch (initial contents), the recorded
call list, and the contents of every written tensor after the method returned.
tests/test_caller_trace.py replays the call list through the installed drop-in
modules on a GPU and through the oracle on CPU.  The reference source itself is
not stored.

Two things the shipped reference leaves undone are filled in here, as the
intended semantics: ``lora_ids`` (all zeros as shipped, model_rpc.py:273) holds
the adapter of each problem, and ``rank_counts`` (a module-level constant tensor
of 64s, req_queue.py:23-33) holds each problem's rank.  output_counts and
start_ids come from the reference's own set_sgmm_args.
"""
from __future__ import annotations

import argparse
import ast
import json
import logging
import os
import sys
import textwrap
import time
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from tests.helpers import (build_tables, fill_pool_a, fill_pool_b, oracle_dispatch_bgmv,  # noqa: E402
                           oracle_dispatch_sgmm, rand_lora)
from tests.golden.make_golden import _Batch, _Self, cuda_to_cpu, load_set_sgmm_args  # noqa: E402

METHODS = ["_lora_get_qkv", "_lora_get_o", "_batch_lora_get_qkv", "_batch_lora_get_o"]


class _TorchProxy:
    """torch, except that torch.cuda.synchronize() does nothing (no GPU here)."""
    cuda = types.SimpleNamespace(synchronize=lambda *a, **k: None)

    def __getattr__(self, name):
        return getattr(torch, name)


def load_callers(ref, ns):
    path = os.path.join(ref, "valora/models/peft/lora_unordered_batch_infer.py")
    src = open(path).read()
    tree = ast.parse(src)
    found = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in METHODS:
            found[node.name] = node
    for name in METHODS:
        exec(textwrap.dedent(ast.get_source_segment(src, found[name])), ns)
    return {name: ns[name] for name in METHODS}


class Recorder:
    """Names tensors by the storage they live in and records calls.  A tensor's contents
    are captured when a call first touches it; if the method's own code changed a tensor
    between two calls (a base projection copied into the KV cache, a correction added to
    q), that is recorded as a host write, so that replaying the list reproduces the run."""

    def __init__(self):
        self.names = {}          # storage data_ptr -> name
        self.base = {}           # name -> flat tensor over the whole storage
        self.shadow = {}         # name -> contents as the recorded calls leave them
        self.arrays = {}         # fixture arrays: init/<name>, write<k>/<name>
        self.calls = []
        self.written = set()
        self.n_tmp = 0

    def register(self, name, t):
        st = t.untyped_storage()
        flat = torch.empty(0, dtype=t.dtype).set_(st, 0, (st.nbytes() // t.element_size(),))
        self.names[st.data_ptr()] = name
        self.base[name] = flat

    def describe(self, t, touch=True):
        key = t.untyped_storage().data_ptr()
        if key not in self.names:
            self.n_tmp += 1
            self.register(f"tmp{self.n_tmp}", t)
        name = self.names[key]
        if touch:
            now = self.base[name]
            if name not in self.shadow:
                self.arrays[f"init/{name}"] = _to_np(now)
            elif not torch.equal(now, self.shadow[name]):
                self.arrays[f"write{len(self.calls)}/{name}"] = _to_np(now)
                self.calls.append({"fn": "host_write", "t": name, "array": f"write{len(self.calls)}/{name}"})
            self.shadow[name] = now.clone()
        return {"t": name, "off": int(t.storage_offset()), "shape": list(t.shape), "stride": list(t.stride())}

    def record(self, fn, args, out_index=0):
        rec = []
        for a in args:
            if isinstance(a, torch.Tensor):
                rec.append(self.describe(a))
            elif a is None:
                rec.append({"none": True})
            else:
                rec.append({"i": int(a)})
        self.calls.append({"fn": fn, "args": rec})
        self.written.add(rec[out_index]["t"])
        return rec[out_index]["t"]

    def after(self, out_name):
        self.shadow[out_name] = self.base[out_name].clone()


def _to_np(t):
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def build_scene(set_sgmm_args, is_prefill, seed):
    """One layer of a small model and one batch, as the reference's forward() leaves them
    in `self` before it calls the per-layer methods (lora_unordered_batch_infer.py:238-343)."""
    dtype = torch.float16
    H, heads = 128, 4
    ranks = [8, 32, 16]
    dirs = ["ad0", "ad1", "ad2"]
    if is_prefill:
        req_ad, req_len = [1, 0, 2, 1, 1, 0], [17, 40, 1, 1, 21, 9]
    else:
        req_ad, req_len = [2, 2, 0, 1, 1, 1, 0, 2, 1], [1] * 9
    g = torch.Generator().manual_seed(seed)
    A, B = rand_lora(ranks, H, H, dtype, n_slots=4, seed=seed, wstd=0.05)
    a_start, a_len, a_loc, total = build_tables(ranks, 4, shuffle=True, contiguous_slots=True, seed=seed)
    key_buffer = fill_pool_a(A, ranks, a_start, a_loc, total, H, dtype).view(1, total, heads, H // heads)
    value_buffer = fill_pool_b(B, ranks, a_start, a_loc, total, H, dtype, layout="rows").view(1, total, heads, H // heads)
    # the problem table: counts and offsets from the reference's own host packer
    with cuda_to_cpu():
        batch = _Batch([dirs[a] for a in req_ad], req_len)
        output_counts, _, start_ids = set_sgmm_args(_Self(dirs), batch, is_prefill, None)
    P = batch.num_problems[0]
    tok = np.repeat(req_ad, req_len).astype(np.int64)
    rle = oracle.rle_ref(tok, np.asarray(ranks) * 4)
    assert rle["P"] == P and np.array_equal(rle["seg_len"], output_counts[:P].numpy())
    lora_ids = torch.zeros(128, dtype=torch.long)
    lora_ids[:P] = torch.from_numpy(rle["seg_adapter"])
    rank_counts = torch.full((128,), 64, dtype=torch.long)
    rank_counts[:P] = torch.from_numpy(rle["seg_rank"])
    T = int(tok.shape[0])
    max_r = max(ranks)
    W = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(dtype)
    layer_w = types.SimpleNamespace(qkv_weight_=W(H, 3 * H), o_weight_=W(H, H), q_weight_=W(H, H),
                                    k_weight_=W(H, H), v_weight_=W(H, H))
    base_model = types.SimpleNamespace(
        trans_layers_weight=[layer_w],
        layers_infer=[types.SimpleNamespace(embed_dim_=H, tp_q_head_num_=heads)],
        tp_k_head_num_=heads, head_dim_=H // heads)
    req_bins = torch.tensor(req_ad, dtype=torch.long)
    me = types.SimpleNamespace(
        base_model=base_model, scheduler="ours", num_problems=P, delora_index=0, delora_tk_index=0,
        tb_x=64, tb_y=32, tb_z=32, wp_x=32, wp_y=32,
        tb_x_b=64, tb_y_b=64, tb_z_b=32, wp_x_b=64, wp_y_b=64,
        infer_adapter=types.SimpleNamespace(
            a_start=torch.from_numpy(a_start), a_len=torch.from_numpy(a_len), a_loc=torch.from_numpy(a_loc),
            a_scaling=torch.tensor([1.0, 0.5, 2.0]).to(dtype)),
        key_buffer=key_buffer, value_buffer=value_buffer,
        req_bins=req_bins, batch_req_bins=torch.from_numpy(tok),
        output_counts=output_counts, lora_ids=lora_ids, start_ids=start_ids,
        delta=[torch.zeros(T, max_r, dtype=dtype) for _ in range(3)],
        delora_delta=[torch.zeros(T, H, dtype=dtype) for _ in range(3)],
        max_lora_dim=max_r, max_b_seq_len=max(req_len), kv_embed_dim=H, de_length=T // 2)
    acts = types.SimpleNamespace(
        input_embs=torch.randn(T, H, generator=g).to(dtype),
        attn_out=torch.randn(T, H, generator=g).to(dtype),
        cache_k=torch.zeros(T, heads, H // heads, dtype=dtype),
        cache_v=torch.zeros(T, heads, H // heads, dtype=dtype))
    tmp_d = torch.zeros(60 * 128, dtype=torch.int8)
    return me, acts, rank_counts, tmp_d, dict(H=H, ranks=ranks, req_ad=req_ad, req_len=req_len, P=int(P), T=T)


def run_scene(ref, set_sgmm_args, is_prefill, seed):
    me, acts, rank_counts, tmp_d, meta = build_scene(set_sgmm_args, is_prefill, seed)
    rec = Recorder()
    for name, t in (("key_buffer", me.key_buffer), ("value_buffer", me.value_buffer),
                    ("a_start", me.infer_adapter.a_start), ("a_len", me.infer_adapter.a_len),
                    ("a_loc", me.infer_adapter.a_loc), ("a_scaling", me.infer_adapter.a_scaling),
                    ("req_bins", me.req_bins), ("batch_req_bins", me.batch_req_bins),
                    ("output_counts", me.output_counts), ("lora_ids", me.lora_ids), ("start_ids", me.start_ids),
                    ("rank_counts", rank_counts), ("tmp_d", tmp_d),
                    ("delta0", me.delta[0]), ("delta1", me.delta[1]), ("delta2", me.delta[2]),
                    ("input_embs", acts.input_embs), ("attn_out", acts.attn_out),
                    ("cache_k", acts.cache_k), ("cache_v", acts.cache_v)):
        rec.register(name, t)

    def dispatch_sgmm(*args):
        out = rec.record("dispatch_sgmm", args)
        oracle_dispatch_sgmm(*args)
        rec.after(out)

    def dispatch_bgmv(*args):
        out = rec.record("dispatch_bgmv", args)
        oracle_dispatch_bgmv(*args)
        rec.after(out)

    ns = {"torch": _TorchProxy(), "dispatch_sgmm": dispatch_sgmm, "dispatch_bgmv": dispatch_bgmv,
          "rank_counts": rank_counts, "tmp_d": tmp_d, "rotary_emb_fwd": lambda *a, **k: None,
          "logging": logging, "time": time}
    fns = load_callers(ref, ns)
    infer_state = types.SimpleNamespace(position_cos=None, position_sin=None,
                                        b_seq_len=torch.tensor(meta["req_len"]))
    returned = {}
    with torch.no_grad():
        if is_prefill:
            q = fns["_lora_get_qkv"](me, 0, acts.input_embs, acts.cache_k, acts.cache_v, infer_state)
            mark = len(rec.calls)
            o = fns["_lora_get_o"](me, 0, acts.attn_out, infer_state)
        else:
            q = fns["_batch_lora_get_qkv"](me, 0, acts.input_embs, acts.cache_k, acts.cache_v, infer_state)
            mark = len(rec.calls)
            o = fns["_batch_lora_get_o"](me, 0, acts.attn_out, infer_state)
    returned["q"] = rec.describe(q, touch=False)
    returned["o"] = rec.describe(o, touch=False)
    final = {name: _to_np(rec.base[name]) for name in sorted(rec.written)}
    return rec, returned, final, meta, mark


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    torch.set_num_threads(1)
    set_sgmm_args = load_set_sgmm_args(args.reference)
    doc, arrays = {"scenes": {}}, {}
    for tag, is_prefill, seed in (("prefill", True, 41), ("decode", False, 43)):
        rec, returned, final, meta, mark = run_scene(args.reference, set_sgmm_args, is_prefill, seed)
        doc["scenes"][tag] = {
            "methods": ["_lora_get_qkv", "_lora_get_o"] if is_prefill else ["_batch_lora_get_qkv", "_batch_lora_get_o"],
            "calls_of_first_method": mark, "meta": meta, "returned": returned, "calls": rec.calls,
            "tensors": {n: {"dtype": str(rec.base[n].dtype).replace("torch.", ""), "numel": int(rec.base[n].numel())}
                        for n in rec.shadow},
            "written": sorted(rec.written)}
        for n, a in rec.arrays.items():
            arrays[f"{tag}/{n}"] = a
        for n, a in final.items():
            arrays[f"{tag}/final/{n}"] = a
        print(tag, "calls:", [(c["fn"], c["args"][0]["t"], c["args"][1]["t"], c["args"][7]["i"]) if "args" in c
                              else (c["fn"], c["t"]) for c in rec.calls])
    with open(os.path.join(args.out, "caller_trace.json"), "w") as f:
        json.dump(doc, f, indent=1)
    np.savez_compressed(os.path.join(args.out, "caller_trace.npz"), **arrays)
    print("caller trace written to", args.out)


if __name__ == "__main__":
    main()
