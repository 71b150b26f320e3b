"""CPU restatement of the reference's LoRA arithmetic (test infrastructure only).

Every function cites the reference lines it follows (paths are relative to the
reference project root).  Two numeric flavours are offered where it matters:

* ``fp32`` - inputs are widened to float32, all arithmetic is float32 and the
  float32 result is returned.  This is the truth the CUDA kernels are held to
  (max-abs error <= 1e-2 for fp16/bf16 outputs).
* ``reference`` - intermediate roundings follow the reference kernels (the
  shrink result is rounded to the 16-bit type before the expand reads it, the
  output is rounded once more), for diagnosing differences.
"""
from __future__ import annotations

import numpy as np
import torch


def _as_list(x):
    if isinstance(x, torch.Tensor):
        return [int(v) for v in x.tolist()]
    return [int(v) for v in x]


# ---------------------------------------------------------------------------
# Per-segment torch path: valora/models/bmm/lora_bmm_infer.py:342-352
#   q[start:end, :] += torch.mm(torch.mm(x[start:end], A_i), B_i) * scaling_i
# ---------------------------------------------------------------------------
def ragged_lora_ref(y0, x, A, B, seg_lens, seg_adapters, scalings):
    """In-dtype walk over segments exactly as the reference's torch path does.

    y0 [T, H_out], x [T, H_in]; A[i] is [H_in, r_i], B[i] is [r_i, H_out];
    segment s covers rows [sum(seg_lens[:s]), +seg_lens[s]) and uses adapter
    seg_adapters[s].  Returns a new tensor of y0's dtype.
    """
    y = y0.clone()
    start = 0
    for length, a in zip(_as_list(seg_lens), _as_list(seg_adapters)):
        end = start + length
        if length > 0:
            xs = x[start:end, :]
            y[start:end, :] += torch.mm(torch.mm(xs, A[a]), B[a]) * scalings[a]
        start = end
    return y


def ragged_lora_ref_fp32(y0, x, A, B, seg_lens, seg_adapters, scalings):
    """Same walk with float32 arithmetic on the widened 16-bit inputs."""
    y = y0.float().clone()
    xf = x.float()
    start = 0
    for length, a in zip(_as_list(seg_lens), _as_list(seg_adapters)):
        end = start + length
        if length > 0:
            v = xf[start:end] @ A[a].float()
            y[start:end] += (v @ B[a].float()) * float(scalings[a])
        start = end
    return y


# ---------------------------------------------------------------------------
# test/kernel/vllm_utils.py:100-124 (ref_torch_groupgemm)
# ---------------------------------------------------------------------------
def groupgemm_ref(out_tensor, inputs, lora_weights, lora_indices, seq_lens, scaling, op_type):
    """Segment walk: linear(x_seg, W[idx]) * scaling; 'expand' adds into
    out_tensor, anything else copies.  lora_weights is [n_lora, out, in]."""
    outs = []
    off = 0
    for b, length in enumerate(_as_list(seq_lens)):
        xs = inputs[off:off + length, :]
        off += length
        w = lora_weights[int(lora_indices[b])]
        r = torch.nn.functional.linear(xs, w)
        r = r * scaling
        outs.append(r)
    cat = torch.cat(outs, dim=0)
    if op_type == "expand":
        out_tensor += cat
    else:
        out_tensor.copy_(cat)
    return out_tensor


# ---------------------------------------------------------------------------
# BGMV, pool-addressed: valora/csrc/bgmv/bgmv_impl.cuh
# ---------------------------------------------------------------------------
def bgmv_shrink_ref(y, x, w, a_start, a_len, a_loc, indicies, qkvo, rounding="fp32"):
    """valora/csrc/bgmv/bgmv_impl.cuh:14-149.

    For token b with adapter a = indicies[b], r = a_len[a] // 4 (:35), and each
    j < r: y[b, j] = sum_k x[b, k] * W[a_loc[a_start[a] + r*qkvo + j], k]
    (:37-38, :146-148 - the store OVERWRITES).  Columns j >= r keep their old
    value (:36).  w is [cells, ...] with H_in elements per cell.

    Returns float32 [B, narrow] (rounding="fp32": unrounded sums in the touched
    columns, widened old values elsewhere) or y's dtype (rounding="reference").
    """
    Bn, h_in = x.shape
    wf = w.reshape(w.shape[0], -1).float()
    assert wf.shape[1] == h_in
    xf = x.float()
    out = y.float().clone()
    a_start, a_len, a_loc, indicies = map(_as_list, (a_start, a_len, a_loc, indicies))
    for b in range(Bn):
        a = indicies[b]
        r = a_len[a] // 4
        base = a_start[a] + r * qkvo
        rows = [a_loc[base + j] for j in range(r)]
        out[b, :r] = wf[rows] @ xf[b]
    if rounding == "reference":
        return out.to(y.dtype)
    return out


def bgmv_expand_ref(y, v, w, a_start, a_len, a_loc, indicies, qkvo, scales,
                    layout="punica", rounding="fp32"):
    """valora/csrc/bgmv/bgmv_impl.cuh:152-208.

    For token b with adapter a, r = a_len[a] // 4 and each output o:
      y[b, o] += sum_{k<r} v[b, k] * Wflat[o*r + k] * scale[a]        (:196-207)
    layout="punica": Wflat is the adapter slot read as a flat [H_out, r] array
    spread over r pool cells: flat f = o*r + k lives in cell
    a_loc[a_start[a] + r*qkvo + f // H_out] at offset f % H_out       (:174-179).
    layout="rows": the slot's r cells are rows of B [r, H_out] (cell j = row j,
    addressed through a_loc per row), i.e. element (k, o) at cell k, offset o.
    """
    Bn, narrow = v.shape
    h_out = y.shape[1]
    wf = w.reshape(w.shape[0], -1).float()
    assert wf.shape[1] == h_out
    vf = v.float()
    out = y.float().clone()
    a_start, a_len, a_loc, indicies = map(_as_list, (a_start, a_len, a_loc, indicies))
    sc = scales.float()
    for b in range(Bn):
        a = indicies[b]
        r = a_len[a] // 4
        base = a_start[a] + r * qkvo
        rows = [a_loc[base + j] for j in range(r)]
        slot = wf[rows]                                   # [r, H_out] cells in slot order
        if layout == "punica":
            bt = slot.reshape(h_out, r)                   # flat [H_out, r]
            delta = bt @ vf[b, :r]
        else:
            delta = vf[b, :r] @ slot
        delta = delta * sc[a]
        if rounding == "reference":
            # the kernel rounds the fp32 sum to T, then does a T add (:205-207)
            out[b] = (y[b].float() + delta.to(y.dtype).float())
        else:
            out[b] = out[b] + delta
    if rounding == "reference":
        return out.to(y.dtype)
    return out


# ---------------------------------------------------------------------------
# ATMM grouped GEMM, pool-addressed: atmm/valora/csrc/bgmv/bgmv_impl.cuh
# ---------------------------------------------------------------------------
def _atmm_problem(i, a_start, a_loc, rank_counts, lora_ids, qkvo):
    r = rank_counts[i]
    mem_pos = a_start[lora_ids[i]] + r * qkvo
    return r, a_loc[mem_pos]


def atmm_shrink_ref(y, x, w, a_start, a_loc, qkvo, output_counts, rank_counts,
                    lora_ids, start_ids, num_problems, accumulate=False, rounding="fp32"):
    """atmm/valora/csrc/bgmv/bgmv_impl.cuh:76-99 (problem table) and :142-202.

    Problem i: m = output_counts[i], n = rank_counts[i], k = H_in;
    row0 = a_loc[a_start[lora_ids[i]] + n*qkvo]; the n weight rows are the n
    CONSECUTIVE cells row0 .. row0+n-1 (only a_loc[mem_pos] is read, :89-92);
    X_i = x[start_ids[i] : +m]; Y_i = y[start_ids[i] : +m, :n].
    The reference epilogue is D = 1*X_i W_i^T + 1*Y_i (:174); accumulate=False
    gives the overwrite form V = X A that the operator's contract needs.
    """
    wf = w.reshape(w.shape[0], -1).float()
    out = y.float().clone()
    xf = x.float()
    a_start, a_loc, output_counts, rank_counts, lora_ids, start_ids = map(
        _as_list, (a_start, a_loc, output_counts, rank_counts, lora_ids, start_ids))
    for i in range(int(num_problems)):
        m = output_counts[i]
        r, row0 = _atmm_problem(i, a_start, a_loc, rank_counts, lora_ids, qkvo)
        s = start_ids[i]
        if m <= 0:
            continue
        d = xf[s:s + m] @ wf[row0:row0 + r].T
        if accumulate:
            out[s:s + m, :r] += d
        else:
            out[s:s + m, :r] = d
    if rounding == "reference":
        return out.to(y.dtype)
    return out


def atmm_expand_ref(y, v, w, a_start, a_loc, qkvo, output_counts, rank_counts,
                    lora_ids, start_ids, num_problems, scales=None, rounding="fp32"):
    """atmm/valora/csrc/bgmv/bgmv_impl.cuh:102-125 and :204-264.

    Problem i: k = rank_counts[i], n = H_out; row0 as in the shrink; the k
    consecutive cells from row0 are the rows of B [k, H_out] (row-major, ld =
    H_out, :121-123); Y_i += V_i[:, :k] B.  The reference epilogue uses
    alpha = 1 (no adapter scale); scales (indexed by adapter id) is the
    operator-contract extension, applied in fp32 before the single rounding.
    """
    wf = w.reshape(w.shape[0], -1).float()
    out = y.float().clone()
    vf = v.float()
    a_start, a_loc, output_counts, rank_counts, lora_ids, start_ids = map(
        _as_list, (a_start, a_loc, output_counts, rank_counts, lora_ids, start_ids))
    for i in range(int(num_problems)):
        m = output_counts[i]
        r, row0 = _atmm_problem(i, a_start, a_loc, rank_counts, lora_ids, qkvo)
        s = start_ids[i]
        if m <= 0:
            continue
        d = vf[s:s + m, :r] @ wf[row0:row0 + r]
        if scales is not None:
            d = d * float(scales[lora_ids[i]])
        out[s:s + m] += d
    if rounding == "reference":
        return out.to(y.dtype)
    return out


def max_abs_err(a, b):
    return float((a.float() - b.float()).abs().max()) if a.numel() else 0.0


def np_i64(x):
    return np.asarray(_as_list(x), dtype=np.int64)
