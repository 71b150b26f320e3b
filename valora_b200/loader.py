"""HF PEFT adapter directory -> adapter pool.

Reads what the reference reads (valora/models/peft/layer_weights/hf_load_utils.py:8-47):
`adapter_config.json` for `r` / `lora_alpha`, and every `*.safetensors` file of the
directory, or - if there is none - every `*.bin` except `training_args.bin`.
A LoRA pair of one module of one layer is found by key:

    ...layers.{L}.<...>.{module}.lora_A.weight   [r, in_features]
    ...layers.{L}.<...>.{module}.lora_B.weight   [out_features, r]

(lora_layer_weight.py:372-430 does the same with the fixed module names of its
model).  Into the pool go, per (layer, module):

* A side: r cells = the rows of lora_A.weight, i.e. the rows of A^T
  (lora_layer_weight.py:507-510 packs `A.T.reshape(r, heads, hd)` of its [in, r] copy);
* B side, "rows" layout (what the tensor-core path reads): r cells = the rows of
  B = lora_B.weight^T, [r, out];
* B side, "punica" layout (what the decode BGMV call reads, lora_layer_weight.py:511-516):
  the r cells hold the flat bytes of lora_B.weight [out, r].

Copies to the device go through pinned staging buffers on a stream of the caller's
choice (the reference prefetches adapters on a side stream, infer_adapter.py:154-165).
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, List, Optional, Sequence, Tuple

import torch


def read_adapter(path: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    """(adapter_config.json as a dict, all tensors of the directory on the CPU)."""
    cfg_path = os.path.join(path, "adapter_config.json")
    if not os.path.isfile(cfg_path):
        raise FileNotFoundError(f"{cfg_path} not found")
    with open(cfg_path) as f:
        cfg = json.load(f)
    files = sorted(os.listdir(path))
    st = [f for f in files if f.endswith(".safetensors")]
    bins = [f for f in files if f.endswith(".bin") and f != "training_args.bin"]
    if not st and not bins:
        raise FileNotFoundError("can only support pytorch tensor and safetensors format for weights.")
    weights: Dict[str, torch.Tensor] = {}
    if st:
        from safetensors import safe_open
        for name in st:
            with safe_open(os.path.join(path, name), "pt", "cpu") as fh:
                for k in fh.keys():
                    weights[k] = fh.get_tensor(k)
    else:
        for name in bins:
            weights.update(torch.load(os.path.join(path, name), map_location="cpu", weights_only=True))
    return cfg, weights


def lora_rank(cfg: dict) -> int:
    return int(cfg["r"])


def lora_scaling(cfg: dict) -> float:
    return float(cfg["lora_alpha"]) / float(cfg["r"])


def find_pair(weights: Dict[str, torch.Tensor], layer: int, module: str):
    """(lora_A.weight [r, in] or None, lora_B.weight [out, r] or None) of one module of one layer."""
    pat = re.compile(rf"(^|\.)layers\.{int(layer)}\.(.*\.)?{re.escape(module)}\.lora_([AB])\.(default\.)?weight$")
    a = b = None
    for k, t in weights.items():
        m = pat.search(k)
        if m:
            if m.group(3) == "A":
                a = t
            else:
                b = t
    return a, b


def pool_blocks(weights: Dict[str, torch.Tensor], cfg: dict, layer: int, modules: Sequence[str],
                widths_in: Sequence[int], widths_out: Sequence[int], dtype,
                b_layout: str = "rows") -> Tuple[List[Optional[torch.Tensor]], List[Optional[torch.Tensor]]]:
    """Per module the [r, in] block for the A-side pool and the [r, out] block for the
    B-side pool (None where the adapter does not touch the module: zeros in the pool)."""
    if b_layout not in ("rows", "punica"):
        raise ValueError("b_layout must be 'rows' or 'punica'")
    r = lora_rank(cfg)
    a_blocks: List[Optional[torch.Tensor]] = []
    b_blocks: List[Optional[torch.Tensor]] = []
    for module, h_in, h_out in zip(modules, widths_in, widths_out):
        a, b = find_pair(weights, layer, module)
        if (a is None) != (b is None):
            raise ValueError(f"layer {layer} module {module}: only one of lora_A / lora_B present")
        if a is None:
            a_blocks.append(None)
            b_blocks.append(None)
            continue
        if tuple(a.shape) != (r, h_in) or tuple(b.shape) != (h_out, r):
            raise ValueError(f"layer {layer} module {module}: shapes {tuple(a.shape)} / {tuple(b.shape)} "
                             f"do not match r={r}, in={h_in}, out={h_out}")
        a_blocks.append(a.to(dtype).contiguous())
        if b_layout == "rows":
            b_blocks.append(b.to(dtype).t().contiguous())
        else:
            b_blocks.append(b.to(dtype).contiguous().reshape(r, h_out))
    return a_blocks, b_blocks


def load_into_engine(engine, adapter: int, path: str, modules: Sequence[str],
                     stream: Optional[torch.cuda.Stream] = None):
    """Fill adapter slot `adapter` of a LoraStepEngine from a PEFT directory.  modules[p]
    names the module of the engine's projection p.  The copies run on `stream` (default:
    the current stream) from pinned staging; the returned event marks their end - make the
    compute stream wait for it before the next step that may use the adapter."""
    cfg, weights = read_adapter(path)
    r = lora_rank(cfg)
    if r != engine.ranks[adapter]:
        raise ValueError(f"adapter slot {adapter} holds rank {engine.ranks[adapter]}, the files have r={r}")
    if len(modules) != len(engine.projections):
        raise ValueError("one module name per projection of the engine")
    widths_in = [hi for _, hi, _ in engine.projections]
    widths_out = [ho for _, _, ho in engine.projections]
    dev = engine.device
    stream = stream if stream is not None else torch.cuda.current_stream(dev)
    keep = []                                           # pinned buffers stay alive until the event
    with torch.cuda.stream(stream):
        for layer in range(engine.layers):
            a_blocks, b_blocks = pool_blocks(weights, cfg, layer, modules, widths_in, widths_out, engine.dtype)
            for p in range(len(modules)):
                wa, sa = engine.slot_a[p]
                wb, sb = engine.slot_b[p]
                pa, pb = engine.pool_a[wa], engine.pool_b[wb]
                ca = pa.a_loc[pa.a_start[adapter] + r * sa: pa.a_start[adapter] + r * (sa + 1)]
                cb = pb.a_loc[pb.a_start[adapter] + r * sb: pb.a_start[adapter] + r * (sb + 1)]
                for pool, cells, blk, width in ((pa, ca, a_blocks[p], wa), (pb, cb, b_blocks[p], wb)):
                    if blk is None:
                        pool.buffer[layer].index_fill_(0, cells, 0)
                    else:
                        host = blk.pin_memory()
                        keep.append(host)
                        pool.buffer[layer].index_copy_(0, cells, host.to(dev, non_blocking=True))
        scale = torch.tensor(lora_scaling(cfg), dtype=engine.dtype, device=dev)
        for pools in (engine.pool_a, engine.pool_b):
            for pool in pools.values():
                pool.a_scaling[adapter] = scale
        done = torch.cuda.Event()
        done.record(stream)
    done._keep = keep
    return done
