"""LoraStepEngine: the host-side object a serving loop holds.

It owns the adapter pools (one per side and row width), the activation buffers
of every (layer, projection) problem, the device packer and the step plan, and
runs one step - pack the batch on the device, then shrink + expand of every
problem - without touching the host in between.

In the reference the same work is spread over ModelRpcServer.set_sgmm_args
(valora/server/router/model_infer/model_rpc.py:265-374, host packing),
InferAdapter (valora/server/router/model_infer/infer_adapter.py:94-173, pool
tables) and LoraUnorderedBatchInfer._lora_get_qkv / _lora_get_o
(valora/models/peft/lora_unordered_batch_infer.py:876-1071, 1563-1683: 6-8
operator calls per layer, each followed by a host synchronisation).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import ops, tile_table
from .pool import AdapterPool


class LoraStepEngine:
    def __init__(self, projections: Sequence[Tuple[str, int, int]], ranks: Sequence[int],
                 scalings: Sequence[float], dtype, device, layers: int, max_tokens: int,
                 tile_m: int = 128, mma_min_rows: Optional[int] = None, gather_rows_per_tile: Optional[int] = None,
                 alloc_activations: bool = True, gather_path: str = "mma",
                 wide_gather: Optional[bool] = None, input_of: Optional[Sequence[int]] = None,
                 share_pools_with: Optional["LoraStepEngine"] = None, split_rank_classes: bool = True):
        """input_of[p] = the projection whose activations projection p reads (itself by
        default).  q, k and v of a transformer layer read the same rows, as do gate and
        up (lora_unordered_batch_infer.py:946-965 passes one `input_embs` view to three
        shrinks): with input_of = [0, 0, 0, 3, 4, 4, 6] the engine keeps one X per group,
        the problems of a group point at it, and what the first of them brings in from
        HBM the others find in L2.
        gather_path: "mma" sends rows that are not consecutive in the batch (decode
        tokens) through the tensor-core kernels with gathered rows (up to 128 rows of
        an adapter per tile); "simt" sends them through the gather mat-vec kernels
        (8 rows per tile).  wide_gather: force the wide (True) or the plain (False) form
        of the expand's gather stages for every tile; default: when an adapter below the
        tile table's rank threshold is resident, the form is chosen per tile (wide for
        those adapters), else plain throughout.
        share_pools_with: another engine over the same projections and adapters whose
        adapter pools this one uses instead of allocating its own (a second view of the
        same resident weights, e.g. with other activation buffers)."""
        if gather_path not in ("mma", "simt"):
            raise ValueError("gather_path must be 'mma' or 'simt'")
        # thresholds that are measured, not derived: from the tile table in force
        self.table = tile_table.current()["engine"]
        if mma_min_rows is None:
            mma_min_rows = int(self.table["mma_min_rows"])
        self.gather_path = gather_path
        self.wide_gather = wide_gather
        self.split_rank_classes = split_rank_classes
        if gather_rows_per_tile is None:
            gather_rows_per_tile = int(self.table["gather_rows_per_tile"]) if gather_path == "mma" else 8
        if gather_path == "simt" and gather_rows_per_tile > 8:
            raise ValueError("the SIMT gather kernels take at most 8 rows per tile")
        if gather_path == "mma" and gather_rows_per_tile > 32:
            raise ValueError("a gather tile on the tensor-core path holds at most 32 rows")
        self.projections = list(projections)
        self.input_of = list(range(len(self.projections))) if input_of is None else [int(i) for i in input_of]
        if len(self.input_of) != len(self.projections):
            raise ValueError("input_of needs one entry per projection")
        for p, src in enumerate(self.input_of):
            if not (0 <= src <= p) or self.input_of[src] != src:
                raise ValueError("input_of[p] must name p itself or an earlier projection that reads its own input")
            if self.projections[src][1] != self.projections[p][1]:
                raise ValueError("projections that share an input must have the same input width")
        self.ranks = [int(r) for r in ranks]
        self.dtype, self.device = dtype, torch.device(device)
        self.layers, self.max_tokens = int(layers), int(max_tokens)
        n_ad = len(self.ranks)
        # slot maps: projection p -> (width, slot) on each side
        self.slot_a: Dict[int, Tuple[int, int]] = {}
        self.slot_b: Dict[int, Tuple[int, int]] = {}
        na: Dict[int, int] = {}
        nb: Dict[int, int] = {}
        for p, (_, hi, ho) in enumerate(self.projections):
            self.slot_a[p] = (hi, na.get(hi, 0))
            na[hi] = na.get(hi, 0) + 1
            self.slot_b[p] = (ho, nb.get(ho, 0))
            nb[ho] = nb.get(ho, 0) + 1
        tot_rank = sum(self.ranks)
        if share_pools_with is not None:
            other = share_pools_with
            if other.projections != self.projections or other.ranks != self.ranks or other.layers != self.layers:
                raise ValueError("pools can be shared only between engines over the same projections, adapters and layers")
            self.pool_a, self.pool_b = other.pool_a, other.pool_b
        else:
            self.pool_a = {w: AdapterPool(tot_rank * n + 16, w, n, dtype, self.device, self.layers) for w, n in na.items()}
            self.pool_b = {w: AdapterPool(tot_rank * n + 16, w, n, dtype, self.device, self.layers) for w, n in nb.items()}
            for a in range(n_ad):
                for pools in (self.pool_a, self.pool_b):
                    for pool in pools.values():
                        pool.load_adapter(f"adapter{a}", self.ranks[a], float(scalings[a]),
                                          [[None] * pool.n_slots for _ in range(self.layers)])
        any_pool = next(iter(self.pool_a.values()))
        self.a_len = any_pool.a_len
        self.scales = any_pool.a_scaling
        self.packer = ops.Packer(self.max_tokens, n_ad, self.device, tile_m, mma_min_rows, gather_rows_per_tile)
        self._wide_below = int(tile_table.choice(self.packer.lib, True, max(self.ranks))["wide_gather_below_rank"])
        self.x: List[List[torch.Tensor]] = []
        self.y: List[List[torch.Tensor]] = []
        self.plan: Optional[ops.StepPlan] = None
        self._copy_in = self._copy_out = None
        if alloc_activations:
            for _ in range(self.layers):
                xs: List[torch.Tensor] = []
                for p, (_, hi, _) in enumerate(self.projections):
                    src = self.input_of[p]
                    xs.append(xs[src] if src != p else
                              torch.zeros((self.max_tokens, hi), dtype=dtype, device=self.device))
                self.x.append(xs)
                self.y.append([torch.zeros((self.max_tokens, ho), dtype=dtype, device=self.device)
                               for _, _, ho in self.projections])
            self.build_plan()

    # ---- weights
    def set_adapter_weights(self, layer: int, proj: int, adapter: int, A: torch.Tensor, B: torch.Tensor):
        """A [h_in, r] and B [r, h_out] of one adapter for one projection."""
        r = self.ranks[adapter]
        wa, sa = self.slot_a[proj]
        wb, sb = self.slot_b[proj]
        pa, pb = self.pool_a[wa], self.pool_b[wb]
        ca = pa.a_loc[pa.a_start[adapter] + r * sa: pa.a_start[adapter] + r * (sa + 1)]
        cb = pb.a_loc[pb.a_start[adapter] + r * sb: pb.a_start[adapter] + r * (sb + 1)]
        pa.buffer[layer][ca] = A.to(device=self.device, dtype=self.dtype).T.contiguous()
        pb.buffer[layer][cb] = B.to(device=self.device, dtype=self.dtype)

    def randomize_weights(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        for pools in (self.pool_a, self.pool_b):
            for pool in pools.values():
                for layer in range(self.layers):
                    buf = pool.buffer[layer]
                    buf.copy_((torch.randn(buf.shape, generator=g, device=self.device, dtype=torch.float32) * std).to(self.dtype))
                pool._pristine[:] = False            # free cells no longer read as zeros

    def adapter_weights(self, layer: int, proj: int, adapter: int):
        """(A [h_in, r], B [r, h_out]) read back from the pools."""
        r = self.ranks[adapter]
        wa, sa = self.slot_a[proj]
        wb, sb = self.slot_b[proj]
        pa, pb = self.pool_a[wa], self.pool_b[wb]
        ca = pa.a_loc[pa.a_start[adapter] + r * sa: pa.a_start[adapter] + r * (sa + 1)]
        cb = pb.a_loc[pb.a_start[adapter] + r * sb: pb.a_start[adapter] + r * (sb + 1)]
        return pa.buffer[layer][ca].T.contiguous(), pb.buffer[layer][cb].contiguous()

    # ---- plan
    def build_plan(self):
        problems = []
        for layer in range(self.layers):
            for p in range(len(self.projections)):
                wa, sa = self.slot_a[p]
                wb, sb = self.slot_b[p]
                pa, pb = self.pool_a[wa], self.pool_b[wb]
                problems.append(ops.Problem(self.x[layer][p], self.y[layer][p], pa.buffer[layer],
                                            pb.buffer[layer], pa.a_start, pa.a_loc, pb.a_start,
                                            pb.a_loc, sa, sb))
        self.plan = ops.StepPlan(problems, self.max_tokens)

    # ---- one step, inputs resident in HBM
    def step(self, tok_adapter: torch.Tensor, max_mma_tiles: int = 0, max_gather_tiles: int = 0):
        packed = self.packer.pack(tok_adapter, self.a_len, sort=True)
        self.plan.run(packed, self.scales, max_mma_tiles, max_gather_tiles,
                      phase_mask=ops.PHASE_ALL | self._gather_flag(), max_rank=max(self.ranks))
        return packed

    def _gather_flag(self) -> int:
        if self.gather_path != "mma":
            return 0
        # the form of the expand's gather stages: per tile by the tile table's rank threshold when
        # an adapter below it is resident; forced for every tile when the caller said so
        if self.wide_gather is None:
            wide = ops.STEP_WIDE_GATHER_STAGES if min(self.ranks) < self._wide_below else 0
        else:
            wide = (ops.STEP_WIDE_GATHER_STAGES | ops.STEP_ALL_WIDE_GATHER_STAGES) if self.wide_gather else 0
        # an adapter above rank 64 resident: its consecutive-row tiles need the three-stage ring; they get
        # a launch of their own, and every other tile the four-stage ring (split_rank_classes=False
        # keeps one launch per kernel)
        split = ops.STEP_SPLIT_RANK_CLASSES if (self.split_rank_classes and max(self.ranks) > 64) else 0
        return ops.STEP_GATHER_ON_TENSOR_CORES | wide | split

    def phases(self):
        """(name, phase bit) of the kernel launches of one step, in order."""
        if self.gather_path == "mma":
            return [("shrink", ops.PHASE_SHRINK_MMA), ("expand", ops.PHASE_EXPAND_MMA)]
        return [("shrink_mma", ops.PHASE_SHRINK_MMA), ("shrink_gather", ops.PHASE_SHRINK_GATHER),
                ("expand_mma", ops.PHASE_EXPAND_MMA), ("expand_gather", ops.PHASE_EXPAND_GATHER)]

    def step_timed(self, tok_adapter: torch.Tensor, events):
        """Same work as step(), with a CUDA event recorded on the current stream
        before the packer and after each stage (events: 2 + len(self.phases()))."""
        events[0].record()
        packed = self.packer.pack(tok_adapter, self.a_len, sort=True)
        events[1].record()
        for i, (_, phase) in enumerate(self.phases()):
            self.plan.run(packed, self.scales, 0, 0, phase_mask=phase | self._gather_flag(),
                          max_rank=max(self.ranks))
            events[2 + i].record()
        return packed

    # ---- one step from host buffers (pinned): H2D, step, D2H
    def step_host(self, tok_adapter_host: torch.Tensor, x_host: Sequence[Sequence[torch.Tensor]],
                  y_host: Sequence[Sequence[torch.Tensor]], tok_dev: torch.Tensor,
                  max_mma_tiles: int = 0, max_gather_tiles: int = 0,
                  y_out_host: Optional[Sequence[Sequence[torch.Tensor]]] = None, overlap: bool = True):
        """x_host[layer][p] / y_host[layer][p] are pinned host tensors of T rows; Y0 is
        read from y_host and Y is written to y_out_host (default: back into y_host).
        Returns the bytes copied (h2d, d2h).

        overlap=True pipelines by layer over three streams: a copy-in stream runs
        ahead with the next layers' X and Y0, the current stream packs the batch once
        and runs each layer's problems as soon as its inputs have landed, and a
        copy-out stream drains finished layers - the PCIe link is busy in both
        directions at once.  The current stream waits for the copy-out stream at the
        end, so synchronising it covers the whole step.  overlap=False enqueues
        everything on the current stream."""
        T = tok_adapter_host.numel()
        y_out_host = y_host if y_out_host is None else y_out_host
        n_proj = len(self.projections)
        h2d = d2h = 0
        cur = torch.cuda.current_stream(self.device)
        if overlap:
            if self._copy_in is None:
                self._copy_in = torch.cuda.Stream(self.device)
                self._copy_out = torch.cuda.Stream(self.device)
            s_in, s_out = self._copy_in, self._copy_out
            s_in.wait_stream(cur)          # earlier work on the buffers (a previous step) is done
            s_out.wait_stream(cur)
        else:
            s_in = s_out = cur
        tok_dev[:T].copy_(tok_adapter_host, non_blocking=True)
        h2d += T * 8
        packed = self.packer.pack(tok_dev[:T], self.a_len, sort=True)
        flags = ops.PHASE_ALL | self._gather_flag()
        for layer in range(self.layers):
            with torch.cuda.stream(s_in):
                for p in range(n_proj):
                    if self.input_of[p] == p:          # a shared input crosses the link once
                        self.x[layer][p][:T].copy_(x_host[layer][p][:T], non_blocking=True)
                        h2d += x_host[layer][p][:T].numel() * 2
                    self.y[layer][p][:T].copy_(y_host[layer][p][:T], non_blocking=True)
                    h2d += y_host[layer][p][:T].numel() * 2
            if overlap:
                cur.wait_stream(s_in)      # waits for what s_in holds now: this layer's inputs
                self.plan.run(packed, self.scales, max_mma_tiles, max_gather_tiles, phase_mask=flags,
                              max_rank=max(self.ranks), first=layer * n_proj, count=n_proj)
                s_out.wait_stream(cur)
                with torch.cuda.stream(s_out):
                    for p in range(n_proj):
                        y_out_host[layer][p][:T].copy_(self.y[layer][p][:T], non_blocking=True)
                        d2h += y_out_host[layer][p][:T].numel() * 2
        if overlap:
            cur.wait_stream(s_out)
        else:
            self.plan.run(packed, self.scales, max_mma_tiles, max_gather_tiles, phase_mask=flags,
                          max_rank=max(self.ranks))
            for layer in range(self.layers):
                for p in range(n_proj):
                    y_out_host[layer][p][:T].copy_(self.y[layer][p][:T], non_blocking=True)
                    d2h += y_out_host[layer][p][:T].numel() * 2
        return h2d, d2h
