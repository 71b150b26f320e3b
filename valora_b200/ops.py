"""Host-side operators over libvlr.so: argument checks mirror the reference's
pybind entry points, then raw pointers go through the C ABI on torch's current
stream.  There is no CPU or eager fallback: a missing library or a non-CUDA
tensor raises."""
from __future__ import annotations

import contextlib
import ctypes
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from . import _lib

F16, BF16 = 0, 1
LAYOUT_PUNICA, LAYOUT_ROWS = 0, 1
ATMM_ACCUMULATE_SHRINK, ATMM_APPLY_SCALE, ATMM_FULL_TILES = 1, 2, 4
TILE_INTS, COUNT_INTS = 8, 8
MAX_RANK = 128
PHASE_SHRINK_MMA, PHASE_SHRINK_GATHER, PHASE_EXPAND_MMA, PHASE_EXPAND_GATHER, PHASE_ALL = 1, 2, 4, 8, 15
STEP_GATHER_ON_TENSOR_CORES = 16
STEP_WIDE_GATHER_STAGES = 32
STEP_ALL_WIDE_GATHER_STAGES = 64
STEP_SPLIT_RANK_CLASSES = 128


_NVTX = os.environ.get("VLR_NVTX") == "1"


@contextlib.contextmanager
def _nvtx(name: str):
    """NVTX range around an operator call when VLR_NVTX=1 (for timeline profilers); the
    reference has no ranges of its own around these calls."""
    if not _NVTX:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.bfloat16:
        return BF16
    raise RuntimeError(f"No suitable kernel. dtype={t.dtype}")


def _check_input(t: torch.Tensor, name: str):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _check_dim(t: torch.Tensor, d: int, name: str):
    if t.dim() != d:
        raise RuntimeError(f"{name} must be a {d}D tensor")


def _i64(t: torch.Tensor, name: str):
    if t.dtype != torch.int64:
        raise RuntimeError(f"{name} must be an int64 tensor")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _bind(device):
    lib = _lib.load()
    idx = device.index if device.index is not None else torch.cuda.current_device()
    _lib.check(lib.vlr_set_device(idx), "vlr_set_device")
    return lib


def _common_checks(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies):
    for t, n in ((y, "y"), (x, "x"), (w, "w"), (start_indicies, "start_indicies"),
                 (lora_ranks, "lora_ranks"), (loc_indicies, "loc_indicies"), (indicies, "indicies")):
        _check_input(t, n)
    _check_dim(y, 2, "y")
    _check_dim(x, 2, "x")
    _check_dim(w, 3, "w")
    _check_dim(indicies, 1, "indicies")
    for t, n in ((start_indicies, "start_indicies"), (lora_ranks, "lora_ranks"),
                 (loc_indicies, "loc_indicies"), (indicies, "indicies")):
        _i64(t, n)
    if indicies.size(0) != x.size(0):
        raise RuntimeError(f"CHECK_EQ(indicies.size(0), x.size(0)) failed. {indicies.size(0)} vs {x.size(0)}")
    if y.size(0) != x.size(0):
        raise RuntimeError(f"CHECK_EQ(y.size(0), x.size(0)) failed. {y.size(0)} vs {x.size(0)}")
    if y.dtype != x.dtype or w.dtype != x.dtype:
        raise RuntimeError("y, x and w must share one dtype")


def bgmv(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies, qkvo, lora_scales,
         layout: int = LAYOUT_PUNICA):
    """Decode gather mat-vec; argument meaning and checks of
    valora._kernels.dispatch_bgmv (valora/csrc/lora_ops.cc:76-126)."""
    _common_checks(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies)
    h_in, h_out = x.size(1), y.size(1)
    wide = max(h_in, h_out)
    if w.size(1) * w.size(2) != wide:
        raise RuntimeError(f"No suitable kernel. h_in={h_in} h_out={h_out} dtype={x.dtype}")
    if h_in < h_out:
        _check_input(lora_scales, "lora_scales")
        if lora_scales.dtype != x.dtype:
            raise RuntimeError("lora_scales must have the dtype of x")
    lib = _bind(x.device)
    with _nvtx("vlr.bgmv_shrink" if h_in >= h_out else "vlr.bgmv_expand"):
        rc = lib.vlr_bgmv(_ptr(y), _ptr(x), _ptr(w), _ptr(start_indicies), _ptr(lora_ranks),
                          _ptr(loc_indicies), _ptr(indicies), int(qkvo), _ptr(lora_scales),
                          x.size(0), h_in, h_out, _dtype_code(x), int(layout), _stream(x.device))
    if rc in (-2,):
        raise RuntimeError(f"No suitable kernel. h_in={h_in} h_out={h_out} dtype={x.dtype}")
    _lib.check(rc, "vlr_bgmv")


def atmm(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies, qkvo, lora_scales,
         output_counts, rank_counts, lora_ids, start_ids, tmp_d, num_problems,
         thrd_x=0, thrd_y=0, thrd_z=0, wrap_x=0, wrap_y=0, wrap_z=0, *,
         accumulate_shrink: bool = False, apply_scale: bool = False, full_tiles: bool = False):
    """Ragged grouped shrink / expand; argument meaning and checks of
    atmm_ops.dispatch_bgmv (atmm/valora/csrc/lora_ops.cc:115-186).  The six tile
    integers are accepted and ignored (tile shapes are chosen on the device side
    for sm_100a).  full_tiles: keep 128-row tiles in a shrink with few rows, which
    by default is cut into 32-row tiles."""
    _common_checks(y, x, w, start_indicies, lora_ranks, loc_indicies, indicies)
    for t, n in ((output_counts, "output_counts"), (rank_counts, "rank_counts"),
                 (lora_ids, "lora_ids"), (start_ids, "start_ids")):
        _check_input(t, n)
        _i64(t, n)
    num_problems = int(num_problems)
    for t, n in ((output_counts, "output_counts"), (rank_counts, "rank_counts"),
                 (lora_ids, "lora_ids"), (start_ids, "start_ids")):
        if t.numel() < num_problems:
            raise RuntimeError(f"{n} has fewer than num_problems entries")
    h_in, h_out = x.size(1), y.size(1)
    wide = max(h_in, h_out)
    if w.size(1) * w.size(2) != wide:
        raise RuntimeError(f"No suitable kernel. h_in={h_in} h_out={h_out} dtype={x.dtype}")
    flags = ((ATMM_ACCUMULATE_SHRINK if accumulate_shrink else 0) | (ATMM_APPLY_SCALE if apply_scale else 0)
             | (ATMM_FULL_TILES if full_tiles else 0))
    if apply_scale:
        _check_input(lora_scales, "lora_scales")
        if lora_scales.dtype != x.dtype:
            raise RuntimeError("lora_scales must have the dtype of x")
    lib = _bind(x.device)
    with _nvtx("vlr.atmm_shrink" if h_in >= h_out else "vlr.atmm_expand"):
        rc = lib.vlr_atmm(_ptr(y), _ptr(x), _ptr(w), _ptr(start_indicies), _ptr(lora_ranks),
                          _ptr(loc_indicies), _ptr(indicies), int(qkvo), _ptr(lora_scales),
                          _ptr(output_counts), _ptr(rank_counts), _ptr(lora_ids), _ptr(start_ids),
                          _ptr(tmp_d), 0 if tmp_d is None else tmp_d.numel() * tmp_d.element_size(),
                          num_problems, x.size(0), h_in, h_out, w.size(0), _dtype_code(x), flags,
                          _stream(x.device))
    if rc in (-2,):
        raise RuntimeError(f"No suitable kernel. h_in={h_in} h_out={h_out} dtype={x.dtype}")
    _lib.check(rc, "vlr_atmm")


@dataclass
class Packed:
    """Device-resident result of pack(); nothing is copied to the host."""
    T: int
    perm: torch.Tensor          # int32 [T]
    seg_len: torch.Tensor       # int64 [cap]   = output_counts
    seg_rank: torch.Tensor      # int64 [cap]   = rank_counts
    seg_adapter: torch.Tensor   # int64 [cap]   = lora_ids
    seg_start: torch.Tensor     # int64 [cap+1] = start_ids
    tiles: torch.Tensor         # int32 [tiles_cap, 8]
    gather_rows: torch.Tensor   # int32 [T]
    counts: torch.Tensor        # int32 [8]
    workspace: torch.Tensor

    def host_counts(self):
        c = self.counts.cpu().tolist()
        return dict(P=c[0], n_mma=c[1], n_gather=c[2], n_gather_rows=c[3], status=c[4])


class Packer:
    """Owns the output buffers and the scratch of the device packer for batches
    of up to max_tokens tokens over n_adapters adapters."""

    def __init__(self, max_tokens: int, n_adapters: int, device, tile_m: int = 128,
                 mma_min_rows: int = 16, gather_rows_per_tile: int = 8):
        if not (0 < tile_m <= 128) or mma_min_rows <= 0 or not (0 < gather_rows_per_tile <= 32):
            raise RuntimeError("a tile holds at most 128 consecutive rows or 32 gathered rows")
        self.lib = _bind(torch.device(device))
        self.device = torch.device(device)
        self.max_tokens, self.n_adapters = int(max_tokens), int(n_adapters)
        self.tile_m, self.mma_min_rows, self.grp = tile_m, mma_min_rows, gather_rows_per_tile
        cap = max(self.max_tokens, 1)
        dev = self.device
        self.perm = torch.empty(cap, dtype=torch.int32, device=dev)
        self.seg_len = torch.empty(cap + 1, dtype=torch.int64, device=dev)
        self.seg_rank = torch.empty(cap + 1, dtype=torch.int64, device=dev)
        self.seg_adapter = torch.empty(cap + 1, dtype=torch.int64, device=dev)
        self.seg_start = torch.empty(cap + 1, dtype=torch.int64, device=dev)
        self.tiles = torch.empty((cap, TILE_INTS), dtype=torch.int32, device=dev)
        self.gather_rows = torch.empty(cap, dtype=torch.int32, device=dev)
        self.counts = torch.zeros(COUNT_INTS, dtype=torch.int32, device=dev)
        nbytes = self.lib.vlr_pack_workspace_bytes(self.max_tokens, self.n_adapters)
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=dev)

    def pack(self, tok_adapter: torch.Tensor, a_len: torch.Tensor, sort: bool = True) -> Packed:
        _check_input(tok_adapter, "tok_adapter")
        _check_input(a_len, "a_len")
        _i64(tok_adapter, "tok_adapter")
        _i64(a_len, "a_len")
        T = tok_adapter.numel()
        if T > self.max_tokens or a_len.numel() != self.n_adapters:
            raise RuntimeError("batch exceeds the packer's capacity")
        if tok_adapter.device != self.device or a_len.device != self.device:
            raise RuntimeError("the batch lives on another device than the packer's buffers")
        _bind(self.device)
        with _nvtx("vlr.pack"):
            rc = self._pack(tok_adapter, a_len, T, sort)
        _lib.check(rc, "vlr_pack")
        return Packed(T, self.perm, self.seg_len, self.seg_rank, self.seg_adapter, self.seg_start,
                      self.tiles, self.gather_rows, self.counts, self.workspace)

    def _pack(self, tok_adapter, a_len, T, sort):
        return self.lib.vlr_pack(_ptr(tok_adapter), T, _ptr(a_len), self.n_adapters, int(bool(sort)),
                               self.tile_m, self.mma_min_rows, self.grp, _ptr(self.perm),
                               _ptr(self.seg_len), _ptr(self.seg_rank), _ptr(self.seg_adapter),
                               _ptr(self.seg_start), _ptr(self.tiles), self.tiles.size(0),
                               _ptr(self.gather_rows), _ptr(self.counts), _ptr(self.workspace),
                               self.workspace.numel(), _stream(self.device))


def pack_static(packer: "Packer", tok_adapter: torch.Tensor, a_len: torch.Tensor,
                sort: bool = True) -> Packed:
    """Pack through vlr_pack_static: same outputs as packer.pack(), written into the
    packer's output buffers, but the scratch is the library's built-in array, so
    nothing here or in the library allocates.  For callers that cannot allocate
    (all free HBM already claimed by the serving pool; FFI callers without an
    allocator).  At most 8192 tokens and 1024 adapters; calls must not overlap
    on the GPU; make the first call on a device outside stream capture."""
    _check_input(tok_adapter, "tok_adapter")
    _check_input(a_len, "a_len")
    _i64(tok_adapter, "tok_adapter")
    _i64(a_len, "a_len")
    T = tok_adapter.numel()
    if T > packer.max_tokens or a_len.numel() != packer.n_adapters:
        raise RuntimeError("batch exceeds the packer's output capacity")
    if tok_adapter.device != packer.device or a_len.device != packer.device:
        raise RuntimeError("the batch lives on another device than the packer's buffers")
    _bind(packer.device)           # the built-in scratch is the current device's: make it the packer's
    rc = packer.lib.vlr_pack_static(_ptr(tok_adapter), T, _ptr(a_len), packer.n_adapters,
                                    int(bool(sort)), packer.tile_m, packer.mma_min_rows, packer.grp,
                                    _ptr(packer.perm), _ptr(packer.seg_len), _ptr(packer.seg_rank),
                                    _ptr(packer.seg_adapter), _ptr(packer.seg_start),
                                    _ptr(packer.tiles), packer.tiles.size(0),
                                    _ptr(packer.gather_rows), _ptr(packer.counts),
                                    _stream(packer.device))
    _lib.check(rc, "vlr_pack_static")
    return Packed(T, packer.perm, packer.seg_len, packer.seg_rank, packer.seg_adapter,
                  packer.seg_start, packer.tiles, packer.gather_rows, packer.counts, None)


def fused_proj(y: torch.Tensor, x: torch.Tensor, w_base: torch.Tensor, v: torch.Tensor, wb_pool: torch.Tensor,
               a_start_b: torch.Tensor, a_loc_b: torch.Tensor, slot_b: int, packed: Packed,
               status: Optional[torch.Tensor] = None):
    """y[rows] = x[rows] @ w_base + v[rows, :r] @ B_adapter for the rows of the packed batch's
    consecutive-row tiles: the base projection (torch.mm in the reference,
    lora_unordered_batch_infer.py:885 / :1568) with the LoRA expand as extra steps of the same
    K loop, so y is written once and never read.  v is the shrink result with the adapter
    scale already applied (atmm(..., apply_scale=True) on the shrink).  Rows in gather tiles
    are left alone."""
    for t, n in ((y, "y"), (x, "x"), (w_base, "w_base"), (v, "v"), (wb_pool, "wb_pool")):
        _check_input(t, n)
        if t.dtype != x.dtype:
            raise RuntimeError("y, x, w_base, v and wb_pool must share one dtype")
    for t, n in ((a_start_b, "a_start_b"), (a_loc_b, "a_loc_b")):
        _check_input(t, n)
        _i64(t, n)
    T, h_in = x.shape
    h_out = y.size(1)
    if w_base.shape != (h_in, h_out) or y.size(0) != T or v.size(0) != T or packed.T != T:
        raise RuntimeError("shape mismatch between x, w_base, y, v and the packed batch")
    if wb_pool.numel() % h_out:
        raise RuntimeError("pool size is not a multiple of the row width")
    lib = _bind(x.device)
    with _nvtx("vlr.fused_proj"):
        rc = lib.vlr_fused_proj(_ptr(y), _ptr(x), _ptr(w_base), _ptr(v), v.size(1), _ptr(wb_pool),
                                wb_pool.numel() // h_out, _ptr(a_start_b), _ptr(a_loc_b), int(slot_b),
                                _ptr(packed.tiles), _ptr(packed.counts), 0, T, h_in, h_out, _dtype_code(x),
                                _ptr(status), _stream(x.device))
    _lib.check(rc, "vlr_fused_proj")


def var_len_copy(old_a_start, old_a_len, old_a_location, new_a_start, new_a_location):
    """Index-table compaction; arguments of launch_var_len_copy_triton
    (valora/server/router/model_infer/infer_adapter.py:277-282)."""
    for t, n in ((old_a_start, "old_a_start"), (old_a_len, "old_a_len"),
                 (old_a_location, "old_a_location"), (new_a_start, "new_a_start"),
                 (new_a_location, "new_a_location")):
        _check_input(t, n)
        _i64(t, n)
    lib = _bind(old_a_start.device)
    rc = lib.vlr_var_len_copy(_ptr(old_a_start), _ptr(old_a_len), _ptr(old_a_location),
                              _ptr(new_a_start), _ptr(new_a_location), old_a_start.numel(),
                              _stream(old_a_start.device))
    _lib.check(rc, "vlr_var_len_copy")


class _CProblem(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("y", ctypes.c_void_p), ("wa", ctypes.c_void_p),
                ("wb", ctypes.c_void_p), ("a_start_a", ctypes.c_void_p), ("a_loc_a", ctypes.c_void_p),
                ("a_start_b", ctypes.c_void_p), ("a_loc_b", ctypes.c_void_p),
                ("cells_a", ctypes.c_int64), ("cells_b", ctypes.c_int64),
                ("h_in", ctypes.c_int32), ("h_out", ctypes.c_int32),
                ("slot_a", ctypes.c_int32), ("slot_b", ctypes.c_int32)]


@dataclass
class Problem:
    """One LoRA projection of a step: y += scale * (x A) B over the packed batch."""
    x: torch.Tensor            # [max_rows, h_in]
    y: torch.Tensor            # [max_rows, h_out]
    wa: torch.Tensor           # A-side pool [cells, h_in] (any trailing shape with h_in elements)
    wb: torch.Tensor           # B-side pool [cells, h_out]
    a_start_a: torch.Tensor
    a_loc_a: torch.Tensor
    a_start_b: torch.Tensor
    a_loc_b: torch.Tensor
    slot_a: int
    slot_b: int


class StepPlan:
    """Device-resident table of the problems of a step, built once per set of
    buffers (tensor maps are encoded here, not per step)."""

    def __init__(self, problems: Sequence[Problem], max_rows: int):
        if not problems:
            raise RuntimeError("a step plan needs at least one problem")
        p0 = problems[0]
        self.device = p0.x.device
        self.dtype = p0.x.dtype
        lib = _bind(self.device)
        n = len(problems)
        arr = (_CProblem * n)()
        self.max_h_in = self.max_h_out = 0
        for i, p in enumerate(problems):
            for t, nm in ((p.x, "x"), (p.y, "y"), (p.wa, "wa"), (p.wb, "wb")):
                _check_input(t, nm)
                if t.dtype != self.dtype:
                    raise RuntimeError("all tensors of a plan share one dtype")
            for t, nm in ((p.a_start_a, "a_start_a"), (p.a_loc_a, "a_loc_a"),
                          (p.a_start_b, "a_start_b"), (p.a_loc_b, "a_loc_b")):
                _check_input(t, nm)
                _i64(t, nm)
            h_in, h_out = p.x.size(1), p.y.size(1)
            if p.x.size(0) < max_rows or p.y.size(0) < max_rows:
                raise RuntimeError("x / y hold fewer than max_rows rows")
            if p.wa.numel() % h_in or p.wb.numel() % h_out:
                raise RuntimeError("pool size is not a multiple of the row width")
            arr[i] = _CProblem(p.x.data_ptr(), p.y.data_ptr(), p.wa.data_ptr(), p.wb.data_ptr(),
                               p.a_start_a.data_ptr(), p.a_loc_a.data_ptr(),
                               p.a_start_b.data_ptr(), p.a_loc_b.data_ptr(),
                               p.wa.numel() // h_in, p.wb.numel() // h_out, h_in, h_out,
                               int(p.slot_a), int(p.slot_b))
            self.max_h_in, self.max_h_out = max(self.max_h_in, h_in), max(self.max_h_out, h_out)
        nbytes = lib.vlr_step_plan_bytes(n)
        host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        rc = lib.vlr_step_plan_build(ctypes.cast(arr, ctypes.c_void_p), n, int(max_rows),
                                     _dtype_code(p0.x), ctypes.c_void_p(host.data_ptr()))
        _lib.check(rc, "vlr_step_plan_build")
        # 128-byte aligned device copy (torch allocations are 512-byte aligned)
        self.plan = host.to(self.device)
        self.n, self.max_rows = n, int(max_rows)
        self.problems = list(problems)       # keeps the buffers alive
        self.lib = lib
        self._ws = None

    def workspace(self, T: int) -> torch.Tensor:
        need = self.lib.vlr_lora_step_workspace_bytes(int(T), self.n)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._ws

    def run(self, packed: Packed, scales: torch.Tensor, max_mma_tiles: int = 0,
            max_gather_tiles: int = 0, phase_mask: int = PHASE_ALL, max_rank: int = 0,
            first: int = 0, count: Optional[int] = None, status: Optional[torch.Tensor] = None):
        """Enqueue shrink + expand for the packed batch: of every problem, or of
        problems [first, first + count) (they share the front of the workspace, so
        sub-ranges of one plan must run on one stream).  status: an int32 device
        tensor of one element the kernels OR their status bits into (the caller
        clears and reads it); default: the process-wide word behind device_status()."""
        count = self.n - first if count is None else int(count)
        if first < 0 or count < 1 or first + count > self.n:
            raise RuntimeError("problem range outside the plan")
        _check_input(scales, "scales")
        if scales.dtype != self.dtype:
            raise RuntimeError("scales must have the plan's dtype")
        if packed.T > self.max_rows:
            raise RuntimeError("batch has more rows than the plan's buffers")
        if status is not None:
            _check_input(status, "status")
            if status.dtype != torch.int32 or status.numel() < 1:
                raise RuntimeError("status must be an int32 tensor")
        ws = self.workspace(packed.T)
        plan_ptr = ctypes.c_void_p(self.plan.data_ptr() + first * (self.plan.numel() // self.n))
        _bind(self.device)
        with _nvtx("vlr.lora_step"):
            rc = self.lib.vlr_lora_step(plan_ptr, count, packed.T, _ptr(packed.tiles),
                                        _ptr(packed.gather_rows), int(max_mma_tiles),
                                        int(max_gather_tiles), _ptr(packed.counts), _ptr(scales),
                                        self.max_h_in, self.max_h_out, int(max_rank),
                                        F16 if self.dtype == torch.float16 else BF16, int(phase_mask), _ptr(ws),
                                        ws.numel(), _ptr(status), _stream(self.device))
        _lib.check(rc, "vlr_lora_step")


def device_status(reset: bool = True) -> int:
    """The process-wide device status word (bit 1: a bounded wait gave up, bit 2: a tile
    record was skipped); synchronises the device."""
    return _lib.load().vlr_device_status(int(reset))


def selftest_bounded_wait(budget_cycles: int, device, status: Optional[torch.Tensor] = None) -> int:
    """Run the wait that nothing completes (see vlr_selftest_bounded_wait); returns the
    cycles it took to give up."""
    device = torch.device(device)
    lib = _bind(device)
    waited = torch.zeros(1, dtype=torch.int64, device=device)
    rc = lib.vlr_selftest_bounded_wait(int(budget_cycles), _ptr(status), _ptr(waited), _stream(device))
    _lib.check(rc, "vlr_selftest_bounded_wait")
    return int(waited.item())
