"""Adapter-group sharding on CPU: routing is a partition of the batch, and two
gloo ranks that each serve their own adapters reproduce, row for row, what one
process computes for the whole batch (the oracle is the arithmetic on both
sides - what is under test is the host-side routing, local adapter numbering
and the timing reduction of the multi-GPU path)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from valora_b200 import shard, workloads

H_IN, H_OUT = 64, 96


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _small_box_batch():
    b = workloads.config4(tokens=1024, n_adapters=24)
    return b


def _weights(batch, adapter):
    """A, B of one GLOBAL adapter id: seeded by the id, so any rank can draw them."""
    g = torch.Generator()
    g.manual_seed(1000 + int(adapter))
    r = int(batch.ranks[adapter])
    A = (torch.randn(H_IN, r, generator=g) * 0.05).to(torch.bfloat16)
    B = (torch.randn(r, H_OUT, generator=g) * 0.05).to(torch.bfloat16)
    return A, B


def _activations(batch):
    g = torch.Generator()
    g.manual_seed(7)
    x = torch.randn(batch.T, H_IN, generator=g).to(torch.bfloat16)
    y0 = torch.randn(batch.T, H_OUT, generator=g).to(torch.bfloat16)
    return x, y0


def _serve(batch, world, rank):
    """What GPU `rank` does in a step, on CPU: its rows, its adapters, local ids."""
    s = shard.route(batch.req_adapter, batch.req_len, world, rank)
    own = shard.owned_adapters(batch.n_adapters, world, rank)
    A, B = zip(*[_weights(batch, a) for a in own]) if len(own) else ((), ())
    scal = batch.scalings()[own]
    x, y0 = _activations(batch)
    idx = torch.from_numpy(s.tok_index)
    y = oracle.ragged_lora_ref(y0[idx], x[idx], list(A), list(B), s.req_len, s.req_adapter, scal)
    return s, y


def _exchange_worker(rank, world, port, out_dir):
    """Every rank holds an unsharded slice of the batch; rows go to their adapter's
    owner, get the update there (oracle arithmetic), and come back in place."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batch = _small_box_batch()
        x, y0 = _activations(batch)
        lo, hi = rank * batch.T // world, (rank + 1) * batch.T // world        # this rank's rows of the batch
        tok = torch.from_numpy(batch.tok_adapter[lo:hi].astype(np.int64))
        plan = shard.exchange_plan(tok.numpy(), world)
        xr, ids, rc = shard.dispatch_rows(x[lo:hi], tok, plan)
        yr, ids2, _ = shard.dispatch_rows(y0[lo:hi], tok, plan)
        assert torch.equal(ids, ids2) and np.all(shard.owner(ids.numpy(), world) == rank)
        out = yr.clone()
        sc = batch.scalings()
        for a in np.unique(ids.numpy()):                                       # rows of one adapter, one at a time
            A, B = _weights(batch, int(a))
            rows = torch.nonzero(ids == int(a)).flatten()
            for r in rows.tolist():                                            # per-row: independent of how rows are grouped
                out[r:r + 1] = oracle.ragged_lora_ref(yr[r:r + 1], xr[r:r + 1], [A], [B], [1], [0], [sc[a]])
        back = shard.combine_rows(out, rc, plan)
        np.save(os.path.join(out_dir, f"x{rank}.npy"), back.float().numpy())
    finally:
        dist.destroy_process_group()


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batch = _small_box_batch()
        s, y = _serve(batch, world, rank)
        ms, units = shard.reduce_timing(10.0 + rank, float(s.T))
        gathered = [None] * world
        dist.all_gather_object(gathered, (s.tok_index, y.float().numpy()))
        if rank == 0:
            full = np.zeros((batch.T, H_OUT), np.float32)
            seen = np.zeros(batch.T, np.int32)
            for ti, yy in gathered:
                full[ti] = yy
                seen[ti] += 1
            np.savez(os.path.join(out_dir, "r0.npz"), full=full, seen=seen, ms=ms, units=units)
    finally:
        dist.destroy_process_group()


def test_route_partitions_the_batch_for_every_world_size():
    batch = _small_box_batch()
    for world in (1, 2, 3, 4, 8):
        shards = [shard.route(batch.req_adapter, batch.req_len, world, r) for r in range(world)]
        shard.check_partition(shards, batch.T)
        for s in shards:
            glob = shard.global_id(s.tok_adapter, world, s.rank)
            assert np.array_equal(glob, batch.tok_adapter[s.tok_index])
            assert np.all(shard.owner(glob, world) == s.rank)
            assert np.all(np.diff(s.req_index) > 0)                       # batch order kept
            assert s.T == int(s.req_len.sum())
            # same split as the workload generator's own per-GPU view
            mine = workloads.config4(n_gpus=world, rank=s.rank, tokens=1024, n_adapters=24)
            assert np.array_equal(mine.tok_adapter, glob)
    with pytest.raises(ValueError):
        shard.route(batch.req_adapter, batch.req_len, 2, 2)
    with pytest.raises(ValueError):
        shard.check_partition(shards[:-1], batch.T)


def test_empty_shard_and_no_group():
    s = shard.route(np.array([0, 2, 4]), np.array([3, 1, 2]), 2, 1)       # rank 1 owns no request
    assert s.T == 0 and s.req_index.size == 0 and s.tok_adapter.size == 0
    assert shard.reduce_timing(3.5, 7.0) == (3.5, 7.0)                    # no process group: identity
    assert list(shard.owned_adapters(7, 3, 1)) == [1, 4]


@pytest.mark.timeout(300)
def test_two_gloo_ranks_match_one_process(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "r0.npz")
    batch = _small_box_batch()
    assert np.all(got["seen"] == 1)
    # one process, whole batch, global adapter ids
    AB = [_weights(batch, a) for a in range(batch.n_adapters)]
    x, y0 = _activations(batch)
    want = oracle.ragged_lora_ref(y0, x, [a for a, _ in AB], [b for _, b in AB], batch.req_len,
                                  batch.req_adapter, batch.scalings())
    assert np.array_equal(got["full"], want.float().numpy())              # same rows, same arithmetic: bit-exact
    assert float(got["ms"]) == 11.0 and float(got["units"]) == float(batch.T)


@pytest.mark.timeout(300)
def test_rows_travel_to_their_adapters_owner_and_back(tmp_path):
    world = 2
    mp.spawn(_exchange_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    batch = _small_box_batch()
    x, y0 = _activations(batch)
    sc = batch.scalings()
    want = y0.clone()
    for t in range(batch.T):
        a = int(batch.tok_adapter[t])
        A, B = _weights(batch, a)
        want[t:t + 1] = oracle.ragged_lora_ref(y0[t:t + 1], x[t:t + 1], [A], [B], [1], [0], [sc[a]])
    got = np.concatenate([np.load(tmp_path / f"x{r}.npy") for r in range(world)])
    assert np.array_equal(got, want.float().numpy())


def test_replicating_hot_adapters_evens_the_load():
    b = workloads.config4(tokens=4096, n_adapters=64)
    counts = np.bincount(b.tok_adapter, minlength=64)
    hot = shard.pick_replicated(counts, 4)
    assert len(hot) == 4 and np.all(np.diff(hot) > 0) and counts[hot].min() >= np.sort(counts)[-4]
    for world in (2, 4):
        plain = [shard.route(b.req_adapter, b.req_len, world, r) for r in range(world)]
        bal = [shard.route_with_replication(b.req_adapter, b.req_len, world, r, hot, 64) for r in range(world)]
        shard.check_partition(bal, b.T)
        assert max(s.T for s in bal) <= max(s.T for s in plain)
        base = shard.replicated_base(64, world)
        for s in bal:
            glob_hot = s.tok_adapter >= base
            # replicated adapters get the same local id on every GPU; partitioned ones keep a // world
            assert np.array_equal(hot[s.tok_adapter[glob_hot] - base], b.tok_adapter[s.tok_index][glob_hot])
            part = ~glob_hot
            assert np.array_equal(shard.global_id(s.tok_adapter[part], world, s.rank), b.tok_adapter[s.tok_index][part])
            # the pools' rank table in local numbering matches every token's true adapter rank
            lr = shard.local_ranks(b.ranks, world, s.rank, hot)
            assert np.array_equal(lr[s.tok_adapter], b.ranks[b.tok_adapter[s.tok_index]])
        for r, s in enumerate(plain):
            lr = shard.local_ranks(b.ranks, world, r)
            assert np.array_equal(lr[s.tok_adapter], b.ranks[b.tok_adapter[s.tok_index]])
    odd = shard.local_ranks(np.array([8, 16, 32, 64, 128]), 2, 1, np.array([0]))      # GPU 1 owns 2 of 5
    assert list(odd) == [16, 64, 16, 8]
    assert len(shard.pick_replicated(counts, 0)) == 0
