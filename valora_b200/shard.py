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
groups (NCCL on GPUs, gloo in the CPU tests).  A sharded serving loop uses no
collective besides the barrier around a timed region and the reduction of its
timing; the most popular adapters can be replicated on every GPU to even out
the load under skew (route_with_replication), and a caller that holds an
unsharded token batch can move rows to their adapter's owner and back with one
uneven all-to-all each way (dispatch_rows / combine_rows).
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


# ---------------------------------------------------------------------------
# Hot adapters: replicate the most popular ones on every GPU
# ---------------------------------------------------------------------------
def pick_replicated(adapter_tokens: np.ndarray, top_k: int) -> np.ndarray:
    """Ids of the top_k adapters by token count (ties: lower id first), ascending.
    Replicated adapters live in every GPU's pool; their requests may be served anywhere."""
    adapter_tokens = np.asarray(adapter_tokens, np.int64)
    if top_k <= 0:
        return np.zeros(0, np.int64)
    order = np.lexsort((np.arange(adapter_tokens.shape[0]), -adapter_tokens))
    hot = order[:top_k]
    return np.sort(hot[adapter_tokens[hot] > 0]).astype(np.int64)


def route_balanced(req_adapter: np.ndarray, req_len: np.ndarray, world: int,
                   replicated: np.ndarray) -> np.ndarray:
    """Owner GPU of every request when the adapters in `replicated` are on all GPUs.

    Requests of partitioned adapters go to adapter % world.  Requests of replicated
    adapters are then dealt, longest first (ties: batch order), to the GPU with the
    fewest tokens so far (ties: lowest rank) - a deterministic greedy every rank can
    recompute from the same batch, so no coordination is needed."""
    req_adapter = np.asarray(req_adapter, np.int64)
    req_len = np.asarray(req_len, np.int64)
    dest = owner(req_adapter, world).astype(np.int64)
    hot = np.isin(req_adapter, np.asarray(replicated, np.int64))
    load = np.zeros(int(world), np.int64)
    np.add.at(load, dest[~hot], req_len[~hot])
    idx = np.nonzero(hot)[0]
    for i in idx[np.lexsort((idx, -req_len[idx]))]:
        g = int(np.argmin(load))
        dest[i] = g
        load[g] += req_len[i]
    return dest


def route_with_replication(req_adapter: np.ndarray, req_len: np.ndarray, world: int, rank: int,
                           replicated: np.ndarray, n_adapters: int) -> Shard:
    """route() for a pool where `replicated` adapters exist on every GPU.  Local ids:
    partitioned adapter a -> a // world as before; replicated adapter number j (in
    ascending id order) -> n_local_partitioned + j, where n_local_partitioned is the
    largest partitioned local id any GPU can have plus one (replicated_base)."""
    req_adapter = np.asarray(req_adapter, np.int64)
    req_len = np.asarray(req_len, np.int64)
    replicated = np.sort(np.asarray(replicated, np.int64))
    dest = route_balanced(req_adapter, req_len, world, replicated)
    keep = np.nonzero(dest == rank)[0]
    starts = np.concatenate([[0], np.cumsum(req_len)])[:-1]
    lens = req_len[keep]
    tok_index = (np.concatenate([np.arange(starts[i], starts[i] + req_len[i], dtype=np.int64) for i in keep])
                 if keep.size else np.zeros(0, np.int64))
    ad = req_adapter[keep]
    pos = np.searchsorted(replicated, ad)
    is_hot = (pos < replicated.shape[0]) & (replicated[np.minimum(pos, max(replicated.shape[0] - 1, 0))] == ad) \
        if replicated.size else np.zeros(ad.shape, bool)
    n_part = replicated_base(n_adapters, world)
    loc = np.where(is_hot, n_part + pos, local_id(ad, world)).astype(np.int32)
    return Shard(rank, world, keep.astype(np.int64), loc, lens, tok_index, np.repeat(loc, lens).astype(np.int32))


def local_ranks(adapter_ranks: np.ndarray, world: int, rank: int, replicated: Optional[np.ndarray] = None,
                filler: int = 16) -> np.ndarray:
    """Rank of every LOCAL adapter id of GPU `rank`'s pools: its partitioned adapters at
    a // world, then (with `replicated`) the replicated ones from replicated_base() on, in
    ascending global id - the numbering route() / route_with_replication() use.  Local ids
    no adapter maps to (a GPU that owns one adapter fewer than the others) get `filler`."""
    adapter_ranks = np.asarray(adapter_ranks, np.int64)
    n = adapter_ranks.shape[0]
    own = owned_adapters(n, world, rank)
    if replicated is None:
        return adapter_ranks[own].copy()
    replicated = np.sort(np.asarray(replicated, np.int64))
    base = replicated_base(n, world)
    out = np.full(base + replicated.shape[0], int(filler), np.int64)
    out[:own.shape[0]] = adapter_ranks[own]
    out[base:] = adapter_ranks[replicated]
    return out


def replicated_base(n_adapters: int, world: int) -> int:
    """First local id used for replicated adapters: one past the largest partitioned local id."""
    return (int(n_adapters) + int(world) - 1) // int(world)


# ---------------------------------------------------------------------------
# Unsharded token batches: rows travel to their adapter's owner and back
# ---------------------------------------------------------------------------
@dataclass
class ExchangePlan:
    """How the rows one rank holds are regrouped by destination GPU."""
    send_order: np.ndarray     # [T_local] local row indices, grouped by destination, stable
    send_counts: np.ndarray    # [world] rows sent to each GPU


def exchange_plan(tok_adapter: np.ndarray, world: int) -> ExchangePlan:
    tok_adapter = np.asarray(tok_adapter, np.int64)
    dest = owner(tok_adapter, world)
    order = np.argsort(dest, kind="stable").astype(np.int64)
    return ExchangePlan(order, np.bincount(dest, minlength=int(world)).astype(np.int64))


def dispatch_rows(rows: torch.Tensor, tok_adapter: torch.Tensor, plan: ExchangePlan, group=None):
    """One uneven all_to_all_single of activation rows (and their adapter ids) to the
    GPUs that own their adapters.  Returns (rows_here, adapters_here, recv_counts);
    rows_here is grouped by source rank.  The inverse is combine_rows.  This is the
    only data-path collective the design has, and only for callers that hold an
    unsharded batch; kernels always read local memory."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    # the counts travel on the rows' device: an NCCL group has no CPU backend, gloo has no CUDA one
    send_counts = torch.from_numpy(plan.send_counts).to(rows.device)
    recv_counts = torch.empty(world, dtype=torch.int64, device=rows.device)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    send_counts, recv_counts = send_counts.cpu(), recv_counts.cpu()
    order = torch.from_numpy(plan.send_order).to(rows.device)
    send_rows = rows.index_select(0, order).contiguous()
    send_ids = tok_adapter.index_select(0, order).contiguous()
    n_in = int(recv_counts.sum())
    out_rows = rows.new_empty((n_in,) + tuple(rows.shape[1:]))
    out_ids = tok_adapter.new_empty((n_in,))
    sc, rc = [int(v) for v in send_counts], [int(v) for v in recv_counts]
    dist.all_to_all_single(out_rows, send_rows, output_split_sizes=rc, input_split_sizes=sc, group=group)
    dist.all_to_all_single(out_ids, send_ids, output_split_sizes=rc, input_split_sizes=sc, group=group)
    return out_rows, out_ids, recv_counts.numpy()


def combine_rows(rows_here: torch.Tensor, recv_counts: np.ndarray, plan: ExchangePlan, group=None):
    """Send processed rows back to where they came from and restore the caller's order."""
    import torch.distributed as dist
    sc = [int(v) for v in recv_counts]
    rc = [int(v) for v in plan.send_counts]
    back = rows_here.new_empty((int(plan.send_counts.sum()),) + tuple(rows_here.shape[1:]))
    dist.all_to_all_single(back, rows_here.contiguous(), output_split_sizes=rc, input_split_sizes=sc, group=group)
    out = torch.empty_like(back)
    out.index_copy_(0, torch.from_numpy(plan.send_order).to(back.device), back)
    return out
