"""Merged (single-adapter) mode: fold an adapter into a base weight and take it out again.

    W[h_in, h_out] += sign * scaling * A[h_in, r] @ B[r, h_out]

is the ragged expand with the rows of W in the place of tokens and A in the place of
the shrink result, so it runs on the tensor-core expand kernel as one segment of h_in
rows: W is read and written once, B once.  The reference forms A @ (B * scaling) with
torch.bmm into a temporary and adds it (valora/models/peft/lora_single_batch_infer.py:
103-126 merge, 128-149 unmerge).
"""
from __future__ import annotations

import torch

from . import ops
from .pool import AdapterPool


def _apply(W: torch.Tensor, pool_a: AdapterPool, pool_b: AdapterPool, layer: int, slot_a: int, slot_b: int,
           adapter: int, sign: float):
    if W.dim() != 2 or not W.is_cuda or not W.is_contiguous():
        raise RuntimeError("W must be a contiguous 2-D CUDA tensor [h_in, h_out]")
    h_in, h_out = W.shape
    if pool_a.width != h_in or pool_b.width != h_out:
        raise RuntimeError("pool row widths do not match W")
    if W.dtype != pool_a.dtype:
        raise RuntimeError("W and the pools must share one dtype")
    r = pool_a.ranks[adapter]
    dev = W.device
    cells = pool_a.a_loc[pool_a.a_start[adapter] + r * slot_a: pool_a.a_start[adapter] + r * (slot_a + 1)]
    a_rows = pool_a.buffer[layer][cells]                      # [r, h_in] = A^T
    a = a_rows.t().contiguous()                               # [h_in, r]: plays the shrink result
    scales = pool_b.a_scaling.float().mul(sign).to(W.dtype)
    i64 = dict(dtype=torch.int64, device=dev)
    wb = pool_b.buffer[layer]
    ops.atmm(W, a, wb.view(wb.shape[0], 1, h_out), pool_b.a_start, pool_b.a_len, pool_b.a_loc,
             torch.full((h_in,), adapter, **i64), slot_b, scales,
             torch.tensor([h_in], **i64), torch.tensor([r], **i64), torch.tensor([adapter], **i64),
             torch.tensor([0, h_in], **i64), None, 1, apply_scale=True)


def merge_adapter(W, pool_a, pool_b, layer, slot_a, slot_b, adapter):
    """W += scaling * A @ B for the adapter's slot (A side from pool_a, B side, rows layout, from pool_b)."""
    _apply(W, pool_a, pool_b, layer, slot_a, slot_b, adapter, 1.0)


def unmerge_adapter(W, pool_a, pool_b, layer, slot_a, slot_b, adapter):
    """W -= scaling * A @ B."""
    _apply(W, pool_a, pool_b, layer, slot_a, slot_b, adapter, -1.0)
