"""CPU restatement of the adapter pool's index rules (test infrastructure only)."""
from __future__ import annotations

import numpy as np
import torch


def alloc_ref(mem_state, need_size):
    """MemoryAllocator.alloc, valora/common/mem_allocator.py:30-55.

    mem_state[c] is 1 for a free cell.  The allocation is the first need_size
    free cells in index order - cumsum(mem_state) <= need_size AND free (:36-37)
    - which need not be contiguous.  The chosen cells are marked used in place.
    Raises if fewer than need_size cells are free (:31-32).
    """
    state = np.asarray(mem_state)
    free = int(state.sum())
    if need_size > free:
        raise Exception(f"warn no enough pool space: need_size {need_size} left_size {free}")
    cum = np.cumsum(state.astype(np.int32))
    sel = np.logical_and(cum <= need_size, state == 1)
    index = np.nonzero(sel)[0].astype(np.int64)
    mem_state[index] = 0
    return index


def pack_w_combined_ref(a_homes, b_homes, rank, num_head):
    """LoraLayerWeight.w_combined_home,
    valora/models/peft/layer_weights/lora_layer_weight.py:448-452,506-516.

    a_homes[p] is the A side of slot p as the reference keeps it, [H, r]
    (lora_A.weight transposed, :456-457); b_homes[p] is [r, H] (lora_B.weight
    transposed, :461-463).  Each is packed as home.T.reshape(r, heads, hd), so
    * A side: cell j of the slot holds column j of a_home, i.e. A[:, j];
    * B side: the r cells hold the flat bytes of b_home.T = [H_out, r].
    A missing slot packs as zeros.  Result [2, 4r, heads, hd].
    """
    H = None
    for t in list(a_homes) + list(b_homes):
        if t is not None:
            H = max(t.shape)
            dtype = t.dtype
    hd = H // num_head

    def safe(t):
        if t is None:
            return torch.zeros(rank, num_head, hd, dtype=dtype)
        return t.T.reshape(rank, num_head, hd)

    parts = [safe(t) for t in a_homes] + [safe(t) for t in b_homes]
    return torch.concat(parts).reshape(2, 4 * rank, num_head, hd)


def pool_rows_ref(b_home):
    """The B side in 'rows' form: cell k of the slot is row k of B [r, H_out]
    (what ATMM's expand reads, atmm/valora/csrc/bgmv/bgmv_impl.cuh:114-123)."""
    return b_home.contiguous()


def var_len_copy_ref(old_a_start, old_a_len, old_a_location, new_a_start, new_size):
    """var_len_copy_kernel_triton,
    valora/server/router/model_infer/infer_adapter.py:263-282: for each kept
    adapter i copy old_a_location[old_a_start[i] : +old_a_len[i]] to
    new_a_location[new_a_start[i] : +old_a_len[i]]."""
    old_loc = np.asarray(old_a_location, dtype=np.int64)
    new_loc = np.zeros(int(new_size), np.int64)
    for s, n, d in zip(np.asarray(old_a_start), np.asarray(old_a_len), np.asarray(new_a_start)):
        new_loc[int(d):int(d) + int(n)] = old_loc[int(s):int(s) + int(n)]
    return new_loc
