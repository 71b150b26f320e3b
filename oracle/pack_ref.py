"""CPU restatement of the ragged-batch metadata (test infrastructure only).

Integer work: every result here is compared bit-for-bit with the device packer.
"""
from __future__ import annotations

import numpy as np

FILL_N = 128  # model_rpc.py:267 - the reference's metadata buffers are 128 long


def rle_ref(tok_adapter, a_len):
    """Run-length encode per-token adapter ids in input order.

    Follows count_consecutive_requests, atmm/valora/csrc/bgmv/bgmv_impl.cuh:39-72:
    a new segment starts wherever tok_adapter[i] != tok_adapter[i-1] (:52-63);
    per segment it records the run length (output_counts), the adapter id
    (lora_ids), a_len[id] / 4 (rank_counts) and the index of the run's first
    token (start_ids).  T = 0 gives P = 0 (the reference kernel is undefined
    there).  Returns int64 arrays; seg_start has P+1 entries (last = T), which
    is model_rpc.py:319-320's cat([0], cumsum(output_counts)).
    """
    t = np.asarray(tok_adapter, dtype=np.int64)
    a_len = np.asarray(a_len, dtype=np.int64)
    T = int(t.shape[0])
    if T == 0:
        z = np.zeros(0, np.int64)
        return dict(P=0, seg_len=z, seg_adapter=z, seg_rank=z, seg_start=np.zeros(1, np.int64))
    seg_len, seg_adapter, seg_rank, seg_start = [], [], [], []
    current, start = 1, 0
    for i in range(1, T):
        if t[i] == t[i - 1]:
            current += 1
        else:
            seg_len.append(current)
            seg_rank.append(a_len[t[i - 1]] // 4)
            seg_adapter.append(t[i - 1])
            seg_start.append(start)
            start = i
            current = 1
    seg_len.append(current)
    seg_rank.append(a_len[t[T - 1]] // 4)
    seg_adapter.append(t[T - 1])
    seg_start.append(start)
    seg_start.append(T)
    return dict(P=len(seg_len),
                seg_len=np.asarray(seg_len, np.int64),
                seg_adapter=np.asarray(seg_adapter, np.int64),
                seg_rank=np.asarray(seg_rank, np.int64),
                seg_start=np.asarray(seg_start, np.int64))


def set_sgmm_args_ref(adapter_dirs, input_lengths, is_prefill, merged_adapter_dir=None):
    """Host packer of the reference, filler included.

    Follows ModelRpcServer.set_sgmm_args,
    valora/server/router/model_infer/model_rpc.py:265-374: requests are walked
    in batch order; consecutive requests with the same adapter merge into one
    problem whose length is the sum of their input lengths (prefill, :291-292)
    or their count (decode, :337-338).  output_counts starts as ones(128)
    (:268), start_ids = cat([0], cumsum(output_counts)) (:319-320, :365-366),
    except for a single-request batch, which returns early with
    start_ids = ones(128), start_ids[0] = 0 (:279-285, :325-331).
    The de-LoRA bookkeeping (num_problems[1], and dropping the first problem
    when the leading run belongs to the merged adapter, :313-314, :361-362) is
    kept.  Returns (output_counts, lora_ids, start_ids, num_problems) with
    lora_ids all zero, as shipped (:282, :304, :318 are commented out).
    """
    N = FILL_N
    output_counts = np.ones(N, np.int64)
    lora_ids = np.zeros(N, np.int64)
    start_ids = np.ones(N, np.int64)
    n = len(adapter_dirs)
    num_problems = [0, [0, 0]]
    current_count = 0
    de_lora = 1
    flag = True
    unit = (lambda i: int(input_lengths[i])) if is_prefill else (lambda i: 1)
    req_len = unit(0)
    if n == 1:
        output_counts[0] = req_len
        start_ids[0] = 0
        num_problems[0] = 1
        return output_counts, lora_ids, start_ids, num_problems
    for i in range(1, n):
        if adapter_dirs[i - 1] == adapter_dirs[i]:
            req_len += unit(i)
            de_lora += 1
        else:
            # prefill tests the run that just ended (:294), decode the one that starts (:340)
            probe = adapter_dirs[i - 1] if is_prefill else adapter_dirs[i]
            if probe == merged_adapter_dir and flag:
                num_problems[1][0] = de_lora
                num_problems[1][1] = req_len
            flag = False
            num_problems[0] += 1
            output_counts[current_count] = req_len
            req_len = unit(i)
            current_count += 1
    if adapter_dirs[-1] == merged_adapter_dir and flag:
        num_problems[1][0] = de_lora
        num_problems[1][1] = req_len
    num_problems[0] += 1
    output_counts[current_count] = req_len
    if num_problems[1][1] > 0:
        output_counts = output_counts[1:]
    start_ids = np.concatenate([np.zeros(1, np.int64), np.cumsum(output_counts)])
    if not is_prefill:
        num_problems[1][0] = 0
        num_problems[1][1] = 0
    return output_counts, lora_ids, start_ids, num_problems


def pack_sorted_ref(tok_adapter, adapter_rank, sort=True):
    """Sorted-mode packing: perm = stable argsort of the adapter ids (ties keep
    token order), then the run-length encoding of rle_ref on the permuted ids.
    With sort=False perm is the identity (the reference's order).

    adapter_rank[a] is the rank itself (a_len[a] / 4).
    Returns dict(perm int32[T], P, seg_len/seg_adapter/seg_rank int64[P],
    seg_start int64[P+1]).
    """
    t = np.asarray(tok_adapter, dtype=np.int64)
    T = t.shape[0]
    perm = np.argsort(t, kind="stable").astype(np.int32) if sort else np.arange(T, dtype=np.int32)
    rank4 = np.asarray(adapter_rank, dtype=np.int64) * 4
    out = rle_ref(t[perm], rank4)
    out["perm"] = perm
    return out


TILE_MMA = 0
TILE_GATHER = 1


def tile_schedule_ref(tok_adapter, adapter_rank, perm, tile_m=128, mma_min_rows=16,
                      gather_rows_per_tile=8):
    """Deterministic tile schedule over a packed batch.

    A *chunk* is a maximal run of sorted positions with the same adapter whose
    original rows are consecutive (perm[i+1] == perm[i] + 1).  A chunk of at
    least mma_min_rows rows is cut into tensor-core tiles of up to tile_m rows
    (contiguous rows of the caller's activations, so a tiled bulk copy can
    fetch them).  Rows of shorter chunks are "gather rows": they are appended,
    in sorted order, to gather_rows, and each adapter's gather rows are cut
    into groups of gather_rows_per_tile for the gather mat-vec path.

    Emission order: all tensor-core tiles in sorted order, then all gather
    tiles in sorted order.  Each tile is 8 int32:
      [kind, adapter, rank, first, nrows, segment, sorted_pos, 0]
    where first = original row of the tile's first row (tensor-core tile) or
    the tile's offset into gather_rows (gather tile), and sorted_pos is the
    sorted position of the tile's first row.
    Returns (tiles int32[n,8], gather_rows int32[g], n_mma, n_gather).
    """
    t = np.asarray(tok_adapter, dtype=np.int64)
    perm = np.asarray(perm, dtype=np.int64)
    T = perm.shape[0]
    key = t[perm] if T else np.zeros(0, np.int64)
    rank = np.asarray(adapter_rank, dtype=np.int64)
    mma, gat, gather_rows = [], [], []
    # chunk boundaries
    i = 0
    seg = -1
    pending = None  # (adapter, seg, first_offset, count, sorted_pos) of the open gather group
    short_by_seg = []
    while i < T:
        if i == 0 or key[i] != key[i - 1]:
            seg += 1
        j = i + 1
        while j < T and key[j] == key[i] and perm[j] == perm[j - 1] + 1:
            j += 1
        n = j - i
        a = int(key[i])
        if n >= mma_min_rows:
            for m0 in range(0, n, tile_m):
                mma.append([TILE_MMA, a, int(rank[a]), int(perm[i + m0]), min(tile_m, n - m0),
                            seg, i + m0, 0])
        else:
            for k in range(i, j):
                short_by_seg.append((seg, a, k))
        i = j
    # gather rows are compacted in sorted order; groups never cross a segment
    off = 0
    k = 0
    while k < len(short_by_seg):
        seg_k, a, _ = short_by_seg[k]
        e = k
        while e < len(short_by_seg) and short_by_seg[e][0] == seg_k:
            e += 1
        cnt = e - k
        for g0 in range(0, cnt, gather_rows_per_tile):
            gat.append([TILE_GATHER, a, int(rank[a]), off + g0,
                        min(gather_rows_per_tile, cnt - g0), seg_k, short_by_seg[k + g0][2], 0])
        for q in range(k, e):
            gather_rows.append(int(perm[short_by_seg[q][2]]))
        off += cnt
        k = e
    tiles = np.asarray(mma + gat, dtype=np.int32).reshape(-1, 8)
    return tiles, np.asarray(gather_rows, dtype=np.int32), len(mma), len(gat)
