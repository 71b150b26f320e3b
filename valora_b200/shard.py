"""Adapter-group sharding of the multi-LoRA step over the GPUs of one node.

The step has no exchange between adapters: a token's update reads only its own
adapter's A and B.  So the path shards by adapter group with no data-path
collective - GPU g of G owns the adapters a with a % G == g, holds only their
weights in its pools, and serves the requests routed to them.  The host-side
counterpart in the reference is the adapter-aware request queue
(valora/server/router/cluster_req_queue.py:10-89), which groups requests by
adapter before a batch is formed; the reference itself runs one GPU per model
replica and has no multi-GPU LoRA path.

Everything here is host logic on numpy arrays and torch.distributed process
groups (NCCL on GPUs, gloo in the CPU tests); the only collectives are the
barrier around a timed region and the reduction of its timing.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch


def owner(adapter, world: int):
    """GPU that owns an adapter id (scalar or array)."""
    return np.asarray(adapter) % int(world)


def local_id(adapter, world: int):
    """Index of an adapter inside its owner's pools."""
    return np.asarray(adapter) // int(world)


def global_id(local, world: int, rank: int):
    return np.asarray(local) * int(world) + int(rank)


def owned_adapters(n_adapters: int, world: int, rank: int) -> np.ndarray:
    """Global ids of the adapters GPU `rank` holds, in local-id order."""
    return np.arange(int(rank), int(n_adapters), int(world), dtype=np.int64)


@dataclass
class Shard:
    """The part of one global batch that one GPU serves."""
    rank: int
    world: int
    req_index: np.ndarray      # [n_local_req] positions in the global request list, ascending
    req_adapter: np.ndarray    # [n_local_req] LOCAL adapter id per request
    req_len: np.ndarray        # [n_local_req] tokens per request
    tok_index: np.ndarray      # [T_local] global token row of each local token row
    tok_adapter: np.ndarray    # [T_local] LOCAL adapter id per local token row

    @property
    def T(self) -> int:
        return int(self.tok_index.shape[0])


def route(req_adapter: np.ndarray, req_len: np.ndarray, world: int, rank: int) -> Shard:
    """Requests of the global batch that GPU `rank` serves, in batch order.

    A request is never split: all its tokens go to its adapter's owner, so the
    local batch keeps the consecutive-row runs the tile scheduler looks for."""
    req_adapter = np.asarray(req_adapter, np.int64)
    req_len = np.asarray(req_len, np.int64)
    if req_adapter.shape != req_len.shape:
        raise ValueError("req_adapter and req_len differ in length")
    if world < 1 or not (0 <= rank < world):
        raise ValueError("rank outside the world")
    keep = np.nonzero(owner(req_adapter, world) == rank)[0]
    starts = np.concatenate([[0], np.cumsum(req_len)])[:-1]
    lens = req_len[keep]
    if keep.size:
        tok_index = np.concatenate([np.arange(starts[i], starts[i] + req_len[i], dtype=np.int64) for i in keep])
    else:
        tok_index = np.zeros(0, np.int64)
    loc = local_id(req_adapter[keep], world).astype(np.int32)
    return Shard(rank, world, keep.astype(np.int64), loc, lens, tok_index,
                 np.repeat(loc, lens).astype(np.int32))


def check_partition(shards, n_tokens: int) -> None:
    """Raises unless the shards' token rows are a partition of range(n_tokens)."""
    seen = np.zeros(int(n_tokens), np.int32)
    for s in shards:
        np.add.at(seen, s.tok_index, 1)
    if not np.all(seen == 1):
        raise ValueError("shards do not partition the batch")


def reduce_timing(ms: float, units: float, group=None, device: Optional[torch.device] = None) -> Tuple[float, float]:
    """(max over ranks of ms, sum over ranks of units).  With no initialised
    process group the inputs come back unchanged.  `device` is where the two
    scalars live for the reduction (the rank's GPU under NCCL, CPU under gloo)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(ms), float(units)
    dev = device if device is not None else torch.device("cpu")
    t = torch.tensor([float(ms)], dtype=torch.float64, device=dev)
    u = torch.tensor([float(units)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(u, op=dist.ReduceOp.SUM, group=group)
    return float(t.item()), float(u.item())
