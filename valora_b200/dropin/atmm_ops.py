"""`atmm_ops` replacement: one function, `dispatch_bgmv`, with the 21 positional
arguments of atmm/valora/csrc/lora_ops.cc:115-122.

Semantics kept: direction from h_in vs h_out, problem table on the device,
results written in place, no adapter scale in the expand (the reference's
epilogue alpha is 1).  One deliberate difference: the shrink overwrites its
output instead of adding to it (the reference's beta = 1 only works because its
caller zero-fills the buffer first); `legacy_accumulate=True` restores the add.
Work is enqueued on torch's current stream, not on a private stream."""
from .. import ops

legacy_accumulate = False


def dispatch_bgmv(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies, qkvo, lora_scales,
                  output_counts, rank_counts, lora_ids, start_ids, tmp_d, num_problems,
                  thrd_x, thrd_y, thrd_z, wrap_x, wrap_y, wrap_z):
    ops.atmm(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies, qkvo, lora_scales,
             output_counts, rank_counts, lora_ids, start_ids, tmp_d, num_problems,
             thrd_x, thrd_y, thrd_z, wrap_x, wrap_y, wrap_z,
             accumulate_shrink=legacy_accumulate, apply_scale=False)
