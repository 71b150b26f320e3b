"""`valora._kernels` replacement: `dispatch_bgmv` with the 9 positional
arguments of valora/csrc/lora_ops.cc:76-78.  The B side is read in the
reference's flat [H_out, r] form (valora/csrc/bgmv/bgmv_impl.cuh:174-179)."""
from .. import ops


def dispatch_bgmv(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies, qkvo, lora_scales):
    ops.bgmv(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies, qkvo, lora_scales,
             layout=ops.LAYOUT_PUNICA)
