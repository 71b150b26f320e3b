"""CPU oracle for the multi-LoRA batching operator (TEST INFRASTRUCTURE ONLY).

This package is a CPU restatement, in torch/numpy, of the arithmetic and index
rules of the reference's ATMM / BGMV operators, its ragged-batch metadata and
its adapter pool.  It exists to check the CUDA path.  Only the test-suite, the
smoke check and the benchmark's CPU-baseline leg may import it; the product
package never does.

Pinning: the restatement is checked against outputs produced by running the
reference's own Python (``ref_torch_groupgemm``, ``set_sgmm_args``,
``MemoryAllocator``) in a CPU container; those outputs are committed under
``tests/golden/`` together with the script that made them.  The reference
ships no golden vectors of its own for this path.
"""
from .lora_ref import (  # noqa: F401
    ragged_lora_ref,
    ragged_lora_ref_fp32,
    groupgemm_ref,
    bgmv_shrink_ref,
    bgmv_expand_ref,
    atmm_shrink_ref,
    atmm_expand_ref,
)
from .pack_ref import (  # noqa: F401
    rle_ref,
    set_sgmm_args_ref,
    pack_sorted_ref,
    tile_schedule_ref,
)
from .pool_ref import (  # noqa: F401
    alloc_ref,
    pack_w_combined_ref,
    var_len_copy_ref,
    pool_rows_ref,
)
