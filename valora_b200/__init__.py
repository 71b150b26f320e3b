"""valora_b200: the multi-LoRA batching operator (ragged shrink/expand, decode
gather mat-vec, on-device batch packing, paged adapter pool) for B200 / sm_100a.

The CUDA code lives in libvlr.so behind a C ABI (include/vlr.h); this package is
the thin Python host side.  Importing it does not load the library; the first
operator call does, and fails loudly if the library is missing."""

__all__ = ["ops", "pool", "workloads", "dropin", "build"]
