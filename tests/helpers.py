"""Test helpers: reference-style pools and index tables on CPU tensors."""
from __future__ import annotations

import numpy as np
import torch


def build_tables(ranks, n_slots=4, shuffle=False, contiguous_slots=True, seed=0, spare=7):
    """a_start, a_len (= 4*rank), a_loc for adapters of the given ranks, each
    owning n_slots*rank cells.  shuffle=True permutes the cells of the whole pool
    (paging exercised as in the reference's bench_ops.py); with
    contiguous_slots=True the permutation moves whole adapters only, so every
    slot stays a run of consecutive cells (what the tensor-core path needs)."""
    rng = np.random.default_rng(seed)
    sizes = [n_slots * int(r) for r in ranks]
    total = sum(sizes) + spare
    if not shuffle:
        order = list(range(len(ranks)))
    else:
        order = list(rng.permutation(len(ranks)))
    a_loc_parts = [None] * len(ranks)
    if shuffle and not contiguous_slots:
        cells = rng.permutation(total)[:sum(sizes)]
        off = 0
        for a, sz in enumerate(sizes):
            a_loc_parts[a] = cells[off:off + sz]
            off += sz
    else:
        off = spare // 2
        for a in order:
            a_loc_parts[a] = np.arange(off, off + sizes[a])
            off += sizes[a]
    a_start = np.zeros(len(ranks), np.int64)
    a_start[1:] = np.cumsum(sizes)[:-1]
    a_loc = np.concatenate(a_loc_parts).astype(np.int64)
    a_len = np.asarray([4 * int(r) for r in ranks], np.int64)
    return a_start, a_len, a_loc, total


def fill_pool_a(A, ranks, a_start, a_loc, total, width, dtype, n_slots=None, garbage=True, seed=1):
    """A[p][a] is [H_in, r]: cell j of slot p holds A[:, j] (lora_layer_weight.py:507-510)."""
    n_slots = len(A) if n_slots is None else n_slots
    g = torch.Generator().manual_seed(seed)
    pool = (torch.randn(total, width, generator=g) * (0.5 if garbage else 0.0)).to(dtype)
    for p in range(len(A)):
        for a, r in enumerate(ranks):
            r = int(r)
            cells = a_loc[a_start[a] + r * p: a_start[a] + r * (p + 1)]
            pool[torch.from_numpy(cells)] = A[p][a].T.contiguous().to(dtype)
    return pool


def fill_pool_b(B, ranks, a_start, a_loc, total, width, dtype, layout="rows", garbage=True, seed=2):
    """B[p][a] is [r, H_out].  layout 'rows': cell k = B[k, :].  layout 'punica':
    the slot's r cells hold the flat bytes of B.T = [H_out, r] (lora_layer_weight.py:511-516)."""
    g = torch.Generator().manual_seed(seed)
    pool = (torch.randn(total, width, generator=g) * (0.5 if garbage else 0.0)).to(dtype)
    for p in range(len(B)):
        for a, r in enumerate(ranks):
            r = int(r)
            cells = a_loc[a_start[a] + r * p: a_start[a] + r * (p + 1)]
            blk = B[p][a].to(dtype)
            if layout == "punica":
                blk = blk.T.contiguous().reshape(r, width)
            pool[torch.from_numpy(cells)] = blk
    return pool


def t64(a, device):
    return torch.from_numpy(np.asarray(a, dtype=np.int64)).to(device)


def rand_lora(ranks, h_in, h_out, dtype, n_slots=1, seed=0, wstd=0.02):
    g = torch.Generator().manual_seed(seed)
    A = [[(torch.randn(h_in, int(r), generator=g) * wstd).to(dtype) for r in ranks] for _ in range(n_slots)]
    B = [[(torch.randn(int(r), h_out, generator=g) * wstd).to(dtype) for r in ranks] for _ in range(n_slots)]
    return A, B


OWN_ALLOWANCE = 2e-3


def out_tolerance(ref32, dtype, tol=1e-2):
    """Elementwise bound on |out - ref32| for an output of 16-bit type `dtype`, ref32 being
    the fp32 truth (nothing rounded on the way): tol - or, where the output grid itself is
    coarser than that leaves room for, half an ulp of `dtype` at the reference's magnitude
    plus OWN_ALLOWANCE for the kernels' own error (the shrink result is kept in 16 bits
    between the two kernels, as in the reference; fp32 accumulation order).  Only bf16
    outputs of magnitude 4 and above are affected (half-ulp 0.0156): a correctly rounded
    bf16 result cannot meet 1e-2 there."""
    prec = 8 if dtype == torch.bfloat16 else 11          # significand bits
    mag = ref32.abs().clamp_min(1e-30)
    half_ulp = torch.exp2(torch.floor(torch.log2(mag)) - prec)
    return torch.maximum(torch.full_like(ref32, tol), half_ulp + OWN_ALLOWANCE)


def own_error(got, ref32):
    """The kernel's own error, with the output grid taken out: the largest
    |got - ref32| - half_ulp(ref32) over the elements (0 if none is positive).
    What is left is accumulation order and the 16-bit rounding of the shrink
    result between the two kernels, not the final rounding to the output type."""
    if got.numel() == 0:
        return 0.0
    prec = 8 if got.dtype == torch.bfloat16 else 11
    mag = ref32.abs().clamp_min(1e-30)
    half_ulp = torch.exp2(torch.floor(torch.log2(mag)) - prec)
    return float(((got.float().cpu() - ref32).abs() - half_ulp).clamp_min(0).max())


def oracle_dispatch_sgmm(y, x, w, a_start, a_len, a_loc, indicies, qkvo, scales, output_counts, rank_counts,
                         lora_ids, start_ids, tmp_d, num_problems, *tile_ints, rounding="reference"):
    """The ATMM entry point on CPU with the argument list of atmm_ops.dispatch_bgmv and the
    semantics of the drop-in shim: direction from h_in >= h_out, the shrink overwrites, the
    expand applies no adapter scale (reference epilogue alpha = 1).  y is updated in place
    (rounding="reference") or the fp32 result is returned (rounding="fp32")."""
    import oracle
    assert len(tile_ints) == 6
    fn = oracle.atmm_shrink_ref if x.size(1) >= y.size(1) else oracle.atmm_expand_ref
    r = fn(y, x, w, a_start, a_loc, qkvo, output_counts, rank_counts, lora_ids, start_ids, num_problems,
           rounding=rounding)
    if rounding == "reference":
        y.copy_(r)
    return r


def oracle_dispatch_bgmv(y, x, w, a_start, a_len, a_loc, indicies, qkvo, scales, rounding="reference"):
    """The BGMV entry point on CPU, argument list of valora._kernels.dispatch_bgmv (punica
    layout of the B side, adapter scale applied in the expand)."""
    import oracle
    if x.size(1) >= y.size(1):
        r = oracle.bgmv_shrink_ref(y, x, w, a_start, a_len, a_loc, indicies, qkvo, rounding=rounding)
    else:
        r = oracle.bgmv_expand_ref(y, x, w, a_start, a_len, a_loc, indicies, qkvo, scales, layout="punica",
                                   rounding=rounding)
    if rounding == "reference":
        y.copy_(r)
    return r
