"""vlr_pack_static: the packer entry point that takes no scratch and allocates
nothing, for callers that cannot allocate device memory (a serving step whose
pool already owns the GPU's free memory; FFI callers without an allocator).

Called through the C ABI twice in a row on different batches and compared, bit
for bit, with vlr_pack (caller workspace) on the same inputs.  Collected last so
that a failure here cannot hide the other tests in a stop-at-first-failure run.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _outputs(pk, T):
    c = pk.counts.cpu().numpy().copy()
    P, n_tiles, n_rows = int(c[0]), int(c[1] + c[2]), int(c[3])
    return dict(counts=c, perm=pk.perm[:T].cpu().numpy().copy(),
                seg_len=pk.seg_len[:P].cpu().numpy().copy(), seg_rank=pk.seg_rank[:P].cpu().numpy().copy(),
                seg_adapter=pk.seg_adapter[:P].cpu().numpy().copy(),
                seg_start=pk.seg_start[:P + 1].cpu().numpy().copy(),
                tiles=pk.tiles[:n_tiles].cpu().numpy().copy(),
                gather_rows=pk.gather_rows[:n_rows].cpu().numpy().copy())


def test_pack_static_matches_pack_on_two_calls_in_a_row():
    from valora_b200 import ops, workloads
    rng = np.random.default_rng(5)
    b3 = workloads.config3()
    cases = [(b3.tok_adapter.astype(np.int64), b3.ranks),                       # mixed prefill + decode
             (np.repeat(rng.integers(0, 1024, 1600), rng.integers(1, 12, 1600))[:8192],
              rng.choice([8, 16, 32, 64, 128], size=1024))]                        # at the limits
    results = []
    for tok, ranks in cases:                    # two static calls back to back, no sync in between
        T = tok.shape[0]
        packer = ops.Packer(T, len(ranks), DEV)
        tok_d = torch.from_numpy(tok).to(DEV)
        a_len = torch.from_numpy(np.asarray(ranks, np.int64) * 4).to(DEV)
        results.append((packer, tok_d, a_len, T))
    static_out = []
    for packer, tok_d, a_len, T in results:
        pk = ops.pack_static(packer, tok_d, a_len, sort=True)
        static_out.append(pk)
    torch.cuda.synchronize()
    static_out = [_outputs(pk, r[3]) for pk, r in zip(static_out, results)]
    for (packer, tok_d, a_len, T), got in zip(results, static_out):
        ref = _outputs(packer.pack(tok_d, a_len, sort=True), T)
        assert ref["counts"][4] == 0 and got["counts"][4] == 0
        for k in ref:
            assert np.array_equal(ref[k], got[k]), k
    # and once more in reference order on both batches (scratch holds the other batch's bytes
    # each time; the second is at the limits).  Device memory in use must not move across these
    # calls: the entry point allocates nothing, here or inside the library.
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    got = [ops.pack_static(r[0], r[1], r[2], sort=False) for r in results]
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    got = [_outputs(pk, r[3]) for pk, r in zip(got, results)]
    for (packer, tok_d, a_len, T), g in zip(results, got):
        ref = _outputs(packer.pack(tok_d, a_len, sort=False), T)
        for k in ref:
            assert np.array_equal(ref[k], g[k]), k


def test_pack_static_empty_batch():
    """T = 0: no segments, no tiles, and every count written (the counts array held other
    values before the call)."""
    from valora_b200 import ops
    packer = ops.Packer(16, 4, DEV)
    packer.counts.fill_(77)
    tok = torch.zeros(0, dtype=torch.int64, device=DEV)
    a_len = torch.full((4,), 64, dtype=torch.int64, device=DEV)
    pk = ops.pack_static(packer, tok, a_len)
    assert pk.counts.cpu().tolist() == [0] * 8
    packer.counts.fill_(77)
    assert packer.pack(tok, a_len).counts.cpu().tolist() == [0] * 8


def test_pack_static_refuses_batches_beyond_its_scratch():
    from valora_b200 import ops
    packer = ops.Packer(9000, 8, DEV)
    tok = torch.zeros(8193, dtype=torch.int64, device=DEV)
    a_len = torch.full((8,), 64, dtype=torch.int64, device=DEV)
    with pytest.raises(RuntimeError, match="built-in scratch"):
        ops.pack_static(packer, tok, a_len)
    packer2 = ops.Packer(16, 1025, DEV)
    with pytest.raises(RuntimeError, match="built-in scratch"):
        ops.pack_static(packer2, tok[:16], torch.full((1025,), 64, dtype=torch.int64, device=DEV))
