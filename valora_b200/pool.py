"""Paged adapter weight pool in HBM with the reference's index tables.

One pool holds, for every resident adapter, `n_slots * rank` cells of `width`
elements per layer: slot p occupies cells a_loc[a_start[a] + rank*p : + rank].
The tables keep the reference's meaning (valora/server/router/model_infer/
infer_adapter.py:13-19): a_loc = cell ids, a_start = offset of the adapter in
a_loc, a_len = 4 * rank (the kernels divide by 4), a_scaling = alpha / rank.
Cells are handed out by a bitmap allocator with the semantics of
MemoryAllocator (valora/common/mem_allocator.py:30-75, 201-215): `alloc` takes
the first free cells in index order, `alloc_contiguous` the first free run.
The tensor-core path needs a slot's cells to be consecutive, so adapters are
placed with alloc_contiguous unless contiguous=False is asked for.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import ops


class AdapterPool:
    def __init__(self, cells: int, width: int, n_slots: int, dtype, device, layers: int = 1):
        self.cells, self.width, self.n_slots, self.layers = int(cells), int(width), int(n_slots), int(layers)
        self.dtype, self.device = dtype, torch.device(device)
        # zero-filled so that rows padded up to a multiple of 16 read as zeros
        self.buffer = torch.zeros((self.layers, self.cells, self.width), dtype=dtype, device=self.device)
        self.mem_state = np.ones(self.cells, dtype=np.uint8)       # 1 = free
        self._pristine = np.ones(self.cells, dtype=bool)           # cell never written: still reads as zeros
        self.names: List[str] = []
        self.idx_map: Dict[str, int] = {}
        self.ranks: List[int] = []
        self.a_loc = torch.empty(0, dtype=torch.int64, device=self.device)
        self.a_start = torch.empty(0, dtype=torch.int64, device=self.device)
        self.a_len = torch.empty(0, dtype=torch.int64, device=self.device)
        self.a_scaling = torch.empty(0, dtype=dtype, device=self.device)

    # ---- allocator
    @property
    def can_use_mem_size(self) -> int:
        return int(self.mem_state.sum())

    def alloc(self, need: int) -> np.ndarray:
        if need > self.can_use_mem_size:
            raise Exception(f"warn no enough pool space: need_size {need} left_size {self.can_use_mem_size}")
        cum = np.cumsum(self.mem_state.astype(np.int32))
        sel = np.logical_and(cum <= need, self.mem_state == 1)
        index = np.nonzero(sel)[0].astype(np.int64)
        self.mem_state[index] = 0
        return index

    def alloc_contiguous(self, need: int) -> Optional[np.ndarray]:
        if need > self.can_use_mem_size:
            raise Exception(f"warn no enough pool space: need_size {need} left_size {self.can_use_mem_size}")
        if need == 0:
            return np.zeros(0, np.int64)
        cum = np.concatenate([[0], np.cumsum(self.mem_state.astype(np.int64))])
        run = cum[need:] - cum[:-need]
        starts = np.nonzero(run == need)[0]
        if starts.size == 0:
            return None
        s = int(starts[0])
        self.mem_state[s:s + need] = 0
        return np.arange(s, s + need, dtype=np.int64)

    def free(self, index: np.ndarray):
        self.mem_state[np.asarray(index, dtype=np.int64)] = 1

    # ---- adapters
    def load_adapter(self, name: str, rank: int, scaling: float,
                     slots: Sequence[Sequence[Optional[torch.Tensor]]], contiguous: bool = True) -> int:
        """slots[layer][p] is the [rank, width] block of slot p (None = zeros).
        Returns the adapter's index."""
        if name in self.idx_map:
            return self.idx_map[name]
        need = self.n_slots * rank
        loc = self.alloc_contiguous(need) if contiguous else self.alloc(need)
        if loc is None:
            # enough cells are free but no run of them is long enough: close the holes
            # that offloaded adapters left and try again
            self.defragment()
            loc = self.alloc_contiguous(need)
        if loc is None:
            raise Exception(f"no contiguous run of {need} cells is free")
        loc_t = torch.from_numpy(loc).to(self.device)
        for layer in range(self.layers):
            for p in range(self.n_slots):
                blk = slots[layer][p]
                cells = loc_t[p * rank:(p + 1) * rank]
                if blk is None:
                    # a projection the adapter does not touch contributes nothing: zeros, as the
                    # reference packs them (lora_layer_weight.py safe()).  Freed cells keep the
                    # previous owner's weights, so the fill cannot be skipped.
                    if not self._pristine[loc].all():
                        self.buffer[layer].index_fill_(0, cells, 0)
                else:
                    self.buffer[layer][cells] = blk.to(device=self.device, dtype=self.dtype).reshape(rank, self.width)
        self._pristine[loc] = False
        idx = len(self.names)
        self.idx_map[name] = idx
        self.names.append(name)
        self.ranks.append(rank)
        start = self.a_loc.numel()
        self.a_start = torch.cat([self.a_start, torch.tensor([start], dtype=torch.int64, device=self.device)])
        self.a_len = torch.cat([self.a_len, torch.tensor([4 * rank], dtype=torch.int64, device=self.device)])
        self.a_loc = torch.cat([self.a_loc, loc_t])
        self.a_scaling = torch.cat([self.a_scaling, torch.tensor([scaling], dtype=self.dtype, device=self.device)])
        return idx

    def offload_adapters(self, reserve: Sequence[str]):
        """Drop every adapter not in `reserve`, free its cells and compact the
        index tables on the device (infer_adapter.py:188-252)."""
        keep = [i for i, n in enumerate(self.names) if n in set(reserve)]
        if len(keep) == len(self.names):
            return
        a_start_h, a_len_h = self.a_start.cpu().numpy(), self.a_len.cpu().numpy()
        a_loc_h = self.a_loc.cpu().numpy()
        cells_of = lambda i: self.n_slots * (a_len_h[i] // 4)
        for i in range(len(self.names)):
            if i not in keep:
                self.free(a_loc_h[a_start_h[i]:a_start_h[i] + cells_of(i)])
        if not keep:
            self.__init_tables()
            return
        keep_t = torch.tensor(keep, dtype=torch.int64, device=self.device)
        old_start = self.a_start[keep_t].contiguous()
        new_len = self.a_len[keep_t].contiguous()
        n_cells = (new_len // 4) * self.n_slots
        new_start = torch.zeros_like(n_cells)
        new_start[1:] = torch.cumsum(n_cells, 0)[:-1]
        new_loc = torch.empty(int(n_cells.sum().item()), dtype=torch.int64, device=self.device)
        ops.var_len_copy(old_start, n_cells.contiguous(), self.a_loc, new_start, new_loc)
        self.a_start, self.a_len, self.a_loc = new_start, new_len, new_loc
        self.a_scaling = self.a_scaling[keep_t].contiguous()
        self.names = [self.names[i] for i in keep]
        self.ranks = [self.ranks[i] for i in keep]
        self.idx_map = {n: i for i, n in enumerate(self.names)}

    def defragment(self):
        """Move the resident adapters' cells to the front of the pool, in table order, so
        that the free cells form one run behind them.  Every slot stays a run of
        consecutive cells (what the tensor-core kernels need, as reference ATMM does:
        atmm/valora/csrc/bgmv/bgmv_impl.cuh:89-92); a_loc is rewritten, a_start / a_len
        do not change.  Device-side copies on the current stream, one layer at a time."""
        used = int(self.a_loc.numel())
        if used == 0:
            self.mem_state[:] = 1
            return
        new_loc = torch.arange(used, dtype=torch.int64, device=self.device)
        if not torch.equal(new_loc, self.a_loc):
            for layer in range(self.layers):
                moved = self.buffer[layer].index_select(0, self.a_loc)     # a copy: sources may overlap targets
                self.buffer[layer][:used] = moved
            self.a_loc = new_loc
        self.mem_state[:used] = 0
        self.mem_state[used:] = 1
        self._pristine[:] = False

    def __init_tables(self):
        self.names, self.idx_map, self.ranks = [], {}, []
        self.a_loc = torch.empty(0, dtype=torch.int64, device=self.device)
        self.a_start = torch.empty(0, dtype=torch.int64, device=self.device)
        self.a_len = torch.empty(0, dtype=torch.int64, device=self.device)
        self.a_scaling = torch.empty(0, dtype=self.dtype, device=self.device)

    def layer_view(self, layer: int) -> torch.Tensor:
        """[cells, 1, width] view with the 3-D shape the drop-in entry points check."""
        return self.buffer[layer].view(self.cells, 1, self.width)
