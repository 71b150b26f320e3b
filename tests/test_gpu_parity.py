"""GPU parity: the CUDA path through the C ABI against the CPU oracle on the
same seeded inputs.  Bit-exact for packing and index tables.  Floating point:
every output element is within 1e-2 of the oracle's fp32 result; where the
output's own 16-bit grid is coarser than that (bf16 at |y| >= 4 has a half-ulp
of 0.0156) the bound is the half-ulp of the output type at that magnitude plus
2e-3 for the kernels' own error, which the step tests also assert on its own."""
import numpy as np
import pytest
import torch

import oracle
from valora_b200 import workloads
from tests.helpers import build_tables, fill_pool_a, fill_pool_b, out_tolerance, own_error, rand_lora, t64

pytestmark = pytest.mark.gpu
TOL = 1e-2
# bound on the kernels' own error (accumulation order, the 16-bit shrink result between the
# two kernels), i.e. on what is left of |got - fp32 truth| once half an ulp of the output
# type is taken off: a fifth of TOL
OWN_TOL = 2e-3
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from valora_b200 import ops as _ops
    from valora_b200 import _lib
    _lib.load()
    return _ops


def _err(got, ref32):
    """Largest excess of |got - ref32| over the elementwise tolerance, shifted by
    TOL so that `_err(...) <= TOL` reads 'every element is within its bound'."""
    if got.numel() == 0:
        return 0.0
    excess = (got.float().cpu() - ref32).abs() - out_tolerance(ref32, got.dtype, TOL)
    return float(excess.max()) + TOL


# --------------------------------------------------------------------------- BGMV
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("layout", ["punica", "rows"])
@pytest.mark.parametrize("shuffle", [False, True])
def test_bgmv_multi_rank(ops, dtype, layout, shuffle):
    """Shape of test/kernel/test_kernel_correctness_multi_rank.py: H=1024, two
    adapters of rank 8 and 16, 128 tokens; here both directions and both dtypes."""
    H, ranks, N = 1024, [8, 16], 128
    A, B = rand_lora(ranks, H, H, dtype, n_slots=4, seed=3, wstd=0.1)
    a_start, a_len, a_loc, total = build_tables(ranks, 4, shuffle=shuffle, contiguous_slots=False, seed=5)
    wa = fill_pool_a(A, ranks, a_start, a_loc, total, H, dtype)
    wb = fill_pool_b(B, ranks, a_start, a_loc, total, H, dtype, layout=layout)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(N, H, generator=g).to(dtype)
    idx = torch.tensor([i * len(ranks) // N for i in range(N)])
    scales = torch.tensor([1.0, 0.5]).to(dtype)
    for qkvo in (0, 3):
        v0 = torch.full((N, 16), 7.0).to(dtype)
        ref_v = oracle.bgmv_shrink_ref(v0, x, wa, a_start, a_len, a_loc, idx, qkvo)
        v = v0.to(DEV)
        ops.bgmv(v, x.to(DEV), wa.view(total, 32, H // 32).to(DEV), t64(a_start, DEV), t64(a_len, DEV),
                 t64(a_loc, DEV), idx.to(DEV), qkvo, scales.to(DEV))
        assert _err(v, ref_v) <= TOL
        # columns >= rank keep their old value (bgmv_impl.cuh:36)
        assert torch.all(v[:N // 2, 8:].cpu() == 7.0)
        y0 = torch.randn(N, H, generator=g).to(dtype)
        vin = ref_v.to(dtype)
        ref_y = oracle.bgmv_expand_ref(y0, vin, wb, a_start, a_len, a_loc, idx, qkvo, scales, layout=layout)
        y = y0.to(DEV)
        ops.bgmv(y, vin.to(DEV), wb.view(total, 32, H // 32).to(DEV), t64(a_start, DEV), t64(a_len, DEV),
                 t64(a_loc, DEV), idx.to(DEV), qkvo, scales.to(DEV),
                 layout=ops.LAYOUT_PUNICA if layout == "punica" else ops.LAYOUT_ROWS)
        assert _err(y, ref_y) <= TOL


def test_bgmv_config1(ops):
    """Decode config: 512 tokens, 64 adapters of rank 64, bf16, 4096 -> 4096."""
    b = workloads.config1()
    fl = workloads.make_floats(b)
    H = 4096
    a_start, a_len, a_loc, total = build_tables(b.ranks, 1, shuffle=True, contiguous_slots=False, seed=1)
    wa = fill_pool_a([fl["A"][0]], b.ranks, a_start, a_loc, total, H, b.dtype, garbage=False)
    wb = fill_pool_b([fl["B"][0]], b.ranks, a_start, a_loc, total, H, b.dtype, layout="punica", garbage=False)
    idx = torch.from_numpy(b.tok_adapter.astype(np.int64))
    scales = torch.from_numpy(b.scalings()).to(b.dtype)
    x, y0 = fl["X"][0], fl["Y0"][0]
    v = torch.zeros(b.T, 64, dtype=b.dtype, device=DEV)
    dev = lambda t: t.to(DEV)
    ops.bgmv(v, dev(x), dev(wa).view(total, 32, 128), t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV),
             dev(idx), 0, dev(scales))
    ref_v = oracle.bgmv_shrink_ref(torch.zeros(b.T, 64, dtype=b.dtype), x, wa, a_start, a_len, a_loc, idx, 0)
    assert _err(v, ref_v) <= TOL
    y = dev(y0)
    ops.bgmv(y, v, dev(wb).view(total, 32, 128), t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV),
             dev(idx), 0, dev(scales))
    # end to end against the operator's fp32 truth (no 16-bit rounding of V)
    truth = y0.float().clone()
    for t in range(b.T):
        a = int(idx[t])
        truth[t] += (x[t].float() @ fl["A"][0][a].float()) @ fl["B"][0][a].float() * float(scales[a])
    assert _err(y, truth) <= TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bgmv_many_tokens_mixed_ranks(ops, dtype):
    """2500 tokens (three grouping windows), 37 adapters of ranks 8..128 including
    ranks that are not powers of two, paged cells in random order, uneven adapter
    popularity: every token still gets exactly its own adapter's update."""
    H, N = 768, 2500
    rng = np.random.default_rng(21)
    ranks = rng.choice(np.array([8, 16, 24, 32, 40, 64, 128]), size=37)
    A, B = rand_lora(ranks, H, H, dtype, n_slots=2, seed=8, wstd=0.05)
    a_start, a_len, a_loc, total = build_tables(ranks, 2, shuffle=True, contiguous_slots=False, seed=4)
    wa = fill_pool_a(A, ranks, a_start, a_loc, total, H, dtype)
    wb = fill_pool_b(B, ranks, a_start, a_loc, total, H, dtype, layout="punica")
    g = torch.Generator().manual_seed(12)
    x = torch.randn(N, H, generator=g).to(dtype)
    idx = torch.from_numpy(rng.choice(37, size=N, p=workloads.zipf_probs(37, 1.0))).long()
    scales = (torch.rand(37, generator=g) + 0.5).to(dtype)
    for qkvo in (0, 1):
        v0 = torch.full((N, 128), 3.0).to(dtype)
        ref_v = oracle.bgmv_shrink_ref(v0, x, wa, a_start, a_len, a_loc, idx, qkvo)
        v = v0.to(DEV)
        ops.bgmv(v, x.to(DEV), wa.view(total, 32, H // 32).to(DEV), t64(a_start, DEV), t64(a_len, DEV),
                 t64(a_loc, DEV), idx.to(DEV), qkvo, scales.to(DEV))
        assert _err(v, ref_v) <= TOL
        y0 = torch.randn(N, H, generator=g).to(dtype)
        vin = ref_v.to(dtype)
        ref_y = oracle.bgmv_expand_ref(y0, vin, wb, a_start, a_len, a_loc, idx, qkvo, scales, layout="punica")
        y = y0.to(DEV)
        ops.bgmv(y, vin.to(DEV), wb.view(total, 32, H // 32).to(DEV), t64(a_start, DEV), t64(a_len, DEV),
                 t64(a_loc, DEV), idx.to(DEV), qkvo, scales.to(DEV))
        assert _err(y, ref_y) <= TOL
    assert ops.device_status() == 0


def test_bgmv_rejects_bad_arguments(ops):
    x = torch.zeros(4, 1024, dtype=torch.float16, device=DEV)
    y = torch.zeros(4, 16, dtype=torch.float16, device=DEV)
    w = torch.zeros(64, 32, 32, dtype=torch.float16, device=DEV)
    z = torch.zeros(1, dtype=torch.int64, device=DEV)
    idx = torch.zeros(4, dtype=torch.int64, device=DEV)
    sc = torch.ones(1, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError):
        ops.bgmv(y.cpu(), x, w, z, z, z, idx, 0, sc)                      # not CUDA
    with pytest.raises(RuntimeError):
        ops.bgmv(y, x.t(), w, z, z, z, idx, 0, sc)                        # not contiguous
    with pytest.raises(RuntimeError):
        ops.bgmv(y, x, w, z, z, z, idx[:3], 0, sc)                        # size mismatch
    with pytest.raises(RuntimeError):
        ops.bgmv(y.float(), x.float(), w.float(), z, z, z, idx, 0, sc)    # dtype
    with pytest.raises(RuntimeError):
        ops.bgmv(y, x, w[:, :, :16].contiguous(), z, z, z, idx, 0, sc)    # cell width != h_in


# --------------------------------------------------------------------------- packing
def _pack_and_compare(ops, tok, ranks, sort, tile_m=128, mma_min=16, grp=8):
    tok = np.asarray(tok, np.int64)
    ranks = np.asarray(ranks, np.int64)
    T = tok.shape[0]
    packer = ops.Packer(max(T, 1), len(ranks), DEV, tile_m, mma_min, grp)
    pk = packer.pack(torch.from_numpy(tok).to(DEV), torch.from_numpy(ranks * 4).to(DEV), sort=sort)
    torch.cuda.synchronize()
    c = pk.host_counts()
    ref = oracle.pack_sorted_ref(tok, ranks, sort=sort)
    P = ref["P"]
    assert c["status"] == 0
    assert c["P"] == P
    assert np.array_equal(pk.perm[:T].cpu().numpy(), ref["perm"])
    assert np.array_equal(pk.seg_len[:P].cpu().numpy(), ref["seg_len"])
    assert np.array_equal(pk.seg_rank[:P].cpu().numpy(), ref["seg_rank"])
    assert np.array_equal(pk.seg_adapter[:P].cpu().numpy(), ref["seg_adapter"])
    assert np.array_equal(pk.seg_start[:P + 1].cpu().numpy(), ref["seg_start"])
    tiles, grows, n_mma, n_g = oracle.tile_schedule_ref(tok, ranks, ref["perm"], tile_m, mma_min, grp)
    assert (c["n_mma"], c["n_gather"], c["n_gather_rows"]) == (n_mma, n_g, len(grows))
    assert np.array_equal(pk.tiles[:n_mma + n_g].cpu().numpy(), tiles)
    assert np.array_equal(pk.gather_rows[:len(grows)].cpu().numpy(), grows)
    return pk, ref


@pytest.mark.parametrize("sort", [True, False])
def test_pack_edge_cases(ops, sort):
    ranks = [8, 16, 64, 128, 32]
    _pack_and_compare(ops, [], ranks, sort)
    _pack_and_compare(ops, [3], ranks, sort)
    _pack_and_compare(ops, [2] * 300, ranks, sort)
    _pack_and_compare(ops, [0, 1, 2, 3, 4] * 50, ranks, sort)
    _pack_and_compare(ops, [4] * 15 + [1] * 16 + [4] * 17 + [0] * 129 + [1], ranks, sort)
    _pack_and_compare(ops, [4] * 15 + [1] * 16 + [4] * 17, ranks, sort, tile_m=16, mma_min=4, grp=3)


@pytest.mark.parametrize("cfg", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("sort", [True, False])
def test_pack_configs(ops, cfg, sort):
    b = workloads.CONFIGS[cfg]()
    _pack_and_compare(ops, b.tok_adapter, b.ranks, sort)


def test_pack_random_and_reference_offsets(ops):
    rng = np.random.default_rng(0)
    # 1024 rows is the largest batch packed by one launch, 16384 the largest whose tile pass works in
    # shared memory; above that the workspace is used
    for T, n in ((1000, 7), (5000, 300), (257, 2), (4097, 1024), (1024, 40), (1025, 40),
                 (16384, 1024), (16385, 64), (40000, 2000)):
        ranks = rng.choice([8, 16, 32, 64, 128], size=n)
        # requests of random length, as the engine's repeat_interleave builds them
        req = rng.integers(0, n, size=T // 5 + 1)
        lens = rng.integers(1, 10, size=req.shape[0])
        tok = np.repeat(req, lens)[:T]
        _pack_and_compare(ops, tok, ranks, True)
        pk, ref = _pack_and_compare(ops, tok, ranks, False)
    # reference order reproduces the host packer's offsets: cat([0], cumsum(counts))
    oc, _, si, npb = oracle.set_sgmm_args_ref(["a", "b", "a", "a", "c"], [300, 12, 1, 44, 128], True)
    tok = np.repeat([0, 1, 0, 0, 2], [300, 12, 1, 44, 128])
    pk, ref = _pack_and_compare(ops, tok, [64, 64, 64], False)
    P = npb[0]
    assert np.array_equal(pk.seg_len[:P].cpu().numpy(), oc[:P])
    assert np.array_equal(pk.seg_start[:P + 1].cpu().numpy(), si[:P + 1])


def test_pack_flags_bad_adapter_id(ops):
    packer = ops.Packer(8, 4, DEV)
    tok = torch.tensor([0, 1, 9, 2], dtype=torch.int64, device=DEV)
    pk = packer.pack(tok, torch.full((4,), 64, dtype=torch.int64, device=DEV))
    assert pk.host_counts()["status"] == 1


# --------------------------------------------------------------------------- ATMM (tensor cores)
def _atmm_case(ops, dtype, ranks, seg_len, seg_ad, h, qkvo=0, n_slots=1, seed=0, shuffle=True):
    A, B = rand_lora(ranks, h, h, dtype, n_slots=n_slots, seed=seed)
    a_start, a_len, a_loc, total = build_tables(ranks, n_slots, shuffle=shuffle, contiguous_slots=True, seed=seed)
    wa = fill_pool_a(A, ranks, a_start, a_loc, total, h, dtype)
    wb = fill_pool_b(B, ranks, a_start, a_loc, total, h, dtype, layout="rows")
    T = int(sum(seg_len))
    g = torch.Generator().manual_seed(seed + 100)
    x = torch.randn(T, h, generator=g).to(dtype)
    y0 = torch.randn(T, h, generator=g).to(dtype)
    P = len(seg_len)
    oc = np.asarray(seg_len, np.int64)
    rc = np.asarray([ranks[a] for a in seg_ad], np.int64)
    li = np.asarray(seg_ad, np.int64)
    si = np.concatenate([[0], np.cumsum(oc)]).astype(np.int64)
    R = max(int(r) for r in ranks)
    R = max(R, 16)
    poison = 123.0
    v0 = torch.full((T, R), poison).to(dtype)
    ref_v = oracle.atmm_shrink_ref(v0, x, wa, a_start, a_loc, qkvo, oc, rc, li, si, P)
    idx = torch.zeros(T, dtype=torch.int64)
    scales = torch.tensor([16.0 / r for r in ranks]).to(dtype)
    dev = lambda t: t.to(DEV)
    args_tail = (t64(oc, DEV), t64(rc, DEV), t64(li, DEV), t64(si, DEV), None, P)
    outs = []
    for full_tiles in (False, True):         # 32-row tiles (what a call with few rows gets) and 128-row tiles
        v = dev(v0)
        ops.atmm(v, dev(x), dev(wa).view(total, 1, h), t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV),
                 dev(idx), qkvo, dev(scales), *args_tail, full_tiles=full_tiles)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        assert _err(v, ref_v) <= TOL
        # columns >= rank of each segment are untouched
        vc = v.cpu().float()
        for s in range(P):
            assert torch.all(vc[si[s]:si[s + 1], rc[s]:] == poison)
        outs.append(v.cpu())
    assert torch.equal(outs[0], outs[1])     # same K order, same fp32 accumulation: the cut does not change a bit
    vin = ref_v.to(dtype)
    ref_y = oracle.atmm_expand_ref(y0, vin, wb, a_start, a_loc, qkvo, oc, rc, li, si, P, scales=scales)
    y = dev(y0)
    ops.atmm(y, dev(vin), dev(wb).view(total, 1, h), t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV),
             dev(idx), qkvo, dev(scales), *args_tail, apply_scale=True)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert _err(y, ref_y) <= TOL
    return x, y0, A, B, scales


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_atmm_small(ops, dtype):
    _atmm_case(ops, dtype, [16, 32], [40, 130], [0, 1], 256)


@pytest.mark.parametrize("rank", [8, 16, 32, 64, 128])
def test_atmm_ragged_lengths(ops, rank):
    """every rank x segment lengths around the 32-row box and 128-row tile edges"""
    lens = [1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 513]
    _atmm_case(ops, torch.bfloat16, [rank, rank], lens, [i % 2 for i in range(len(lens))], 512, seed=rank)


def test_atmm_slots_and_mixed_ranks(ops):
    ranks = [8, 16, 24, 64, 128, 40]
    lens = [37, 256, 1, 1, 120, 513, 5, 77]
    ads = [0, 1, 2, 3, 1, 0, 4, 5]
    for qkvo in (0, 2, 3):
        _atmm_case(ops, torch.float16, ranks, lens, ads, 1024, qkvo=qkvo, n_slots=4, seed=qkvo)


def test_atmm_config0(ops):
    """Benchmark config 0 whole: fp16, 4096 -> 4096, ranks {8,16,16,32}, six segments."""
    b = workloads.config0()
    x, y0, A, B, scales = _atmm_case(ops, b.dtype, [int(r) for r in b.ranks], b.req_len.tolist(),
                                     b.req_adapter.tolist(), 4096, seed=0)


def test_atmm_widths_off_the_box_grid(ops):
    """hidden sizes that are multiples of 8 but not of the 64-column box (the copy engine
    zero-fills the ragged last K block / the last output block is stored in part)"""
    for h in (72, 520, 1096):
        _atmm_case(ops, torch.bfloat16, [16, 64, 8], [5, 140, 33, 1], [0, 1, 2, 1], h, seed=h)


def test_atmm_rows_outside_every_problem(ops):
    """A problem table that leaves rows of x / v / y in no problem (before the first
    segment, between segments - inside what would be one 128-row tile or one 32-row copy
    box - and after the last).  Those rows hold NaN everywhere; they must come back bit
    for bit, and must not leak into the rows of the segments next to them."""
    dtype, h = torch.bfloat16, 512
    ranks = [16, 64, 8, 128]
    seg_len = [5, 40, 130, 1, 33, 64]
    seg_ad = [0, 1, 2, 3, 1, 0]
    gaps = [3, 1, 17, 90, 2, 31, 9]              # before segment 0, ..., after the last
    A, B = rand_lora(ranks, h, h, dtype, n_slots=1, seed=77)
    a_start, a_len, a_loc, total = build_tables(ranks, 1, shuffle=True, contiguous_slots=True, seed=7)
    wa = fill_pool_a(A, ranks, a_start, a_loc, total, h, dtype)
    wb = fill_pool_b(B, ranks, a_start, a_loc, total, h, dtype, layout="rows")
    si, pos = [], 0
    for g, m in zip(gaps, seg_len):
        pos += g
        si.append(pos)
        pos += m
    T = pos + gaps[-1]
    inside = np.zeros(T, bool)
    for s0, m in zip(si, seg_len):
        inside[s0:s0 + m] = True
    outside = torch.from_numpy(~inside)
    P = len(seg_len)
    oc = np.asarray(seg_len, np.int64)
    rc = np.asarray([ranks[a] for a in seg_ad], np.int64)
    li = np.asarray(seg_ad, np.int64)
    si = np.asarray(si + [T], np.int64)          # start_ids has P + 1 entries in the reference's buffers
    g = torch.Generator().manual_seed(78)
    x = torch.randn(T, h, generator=g).to(dtype)
    y0 = torch.randn(T, h, generator=g).to(dtype)
    v0 = torch.full((T, 128), 5.0).to(dtype)
    for t in (x, y0, v0):
        t[outside] = float("nan")
    bits = lambda t: t.cpu().view(torch.int16)
    idx = torch.zeros(T, dtype=torch.int64)
    scales = torch.tensor([16.0 / r for r in ranks]).to(dtype)
    dev = lambda t: t.to(DEV)
    tail = (t64(oc, DEV), t64(rc, DEV), t64(li, DEV), t64(si, DEV), None, P)
    ref_v = oracle.atmm_shrink_ref(v0, x, wa, a_start, a_loc, 0, oc, rc, li, si, P)
    for full_tiles in (False, True):
        v = dev(v0)
        ops.atmm(v, dev(x), dev(wa).view(total, 1, h), t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV),
                 dev(idx), 0, dev(scales), *tail, full_tiles=full_tiles)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        assert torch.equal(bits(v)[outside], bits(v0)[outside])
        assert not torch.isnan(v.cpu()[torch.from_numpy(inside)].float()).any()
        assert _err(v[dev(torch.from_numpy(inside))], ref_v[torch.from_numpy(inside)]) <= TOL
    vin = ref_v.to(dtype)
    vin[outside] = float("nan")
    ref_y = oracle.atmm_expand_ref(y0, vin, wb, a_start, a_loc, 0, oc, rc, li, si, P, scales=scales)
    y = dev(y0)
    ops.atmm(y, dev(vin), dev(wb).view(total, 1, h), t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV),
             dev(idx), 0, dev(scales), *tail, apply_scale=True)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(bits(y)[outside], bits(y0)[outside])
    m = torch.from_numpy(inside)
    assert not torch.isnan(y.cpu()[m].float()).any()
    assert _err(y[dev(m)], ref_y[m]) <= TOL


def test_atmm_legacy_accumulate_and_empty(ops):
    dtype, h, ranks = torch.float16, 256, [16]
    A, B = rand_lora(ranks, h, h, dtype, seed=9)
    a_start, a_len, a_loc, total = build_tables(ranks, 1)
    wa = fill_pool_a(A, ranks, a_start, a_loc, total, h, dtype)
    x = torch.randn(50, h).to(dtype)
    v0 = torch.randn(50, 16).to(dtype)
    oc, rc, li, si = [50], [16], [0], [0, 50]
    ref = oracle.atmm_shrink_ref(v0, x, wa, a_start, a_loc, 0, oc, rc, li, si, 1, accumulate=True)
    v = v0.to(DEV)
    idx = torch.zeros(50, dtype=torch.int64, device=DEV)
    ops.atmm(v, x.to(DEV), wa.view(total, 1, h).to(DEV), t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV),
             idx, 0, None, t64(oc, DEV), t64(rc, DEV), t64(li, DEV), t64(si, DEV), None, 1,
             accumulate_shrink=True)
    assert _err(v, ref) <= TOL
    # zero problems: nothing launched, output untouched
    v2 = v0.to(DEV)
    ops.atmm(v2, x.to(DEV), wa.view(total, 1, h).to(DEV), t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV),
             idx, 0, None, t64(oc, DEV), t64(rc, DEV), t64(li, DEV), t64(si, DEV), None, 0)
    assert torch.equal(v2.cpu(), v0)


# --------------------------------------------------------------------------- pool + compaction
def test_var_len_copy_and_pool(ops):
    from valora_b200.pool import AdapterPool
    pool = AdapterPool(cells=512, width=256, n_slots=4, dtype=torch.float16, device=DEV)
    ranks = {"a": 8, "b": 16, "c": 32, "d": 8}
    blocks = {}
    for name, r in ranks.items():
        blocks[name] = [torch.randn(r, 256).half() for _ in range(4)]
        pool.load_adapter(name, r, 16.0 / r, [blocks[name]])
    old = (pool.a_start.cpu().numpy(), pool.a_len.cpu().numpy(), pool.a_loc.cpu().numpy())
    pool.offload_adapters(["a", "c"])
    keep = [0, 2]
    n_cells = old[1][keep]                      # 4 * rank = cells with 4 slots
    new_start = np.concatenate([[0], np.cumsum(n_cells)[:-1]])
    ref = oracle.var_len_copy_ref(old[0][keep], n_cells, old[2], new_start, n_cells.sum())
    assert np.array_equal(pool.a_loc.cpu().numpy(), ref)
    assert pool.names == ["a", "c"]
    assert pool.can_use_mem_size == 512 - 4 * (8 + 32)
    # contents still addressable through the compacted tables
    for i, name in enumerate(pool.names):
        r = ranks[name]
        loc = pool.a_loc[pool.a_start[i]: pool.a_start[i] + 4 * r]
        for p in range(4):
            assert torch.equal(pool.buffer[0][loc[p * r:(p + 1) * r]].cpu(), blocks[name][p])


def test_pool_reuses_freed_cells_and_defragments(ops):
    """Cells freed by an offload keep the old adapter's weights: an adapter that does not
    touch a projection (slot None) must still read zeros there when it lands on them.  And
    when the free cells are plentiful but scattered, loading closes the holes first: every
    resident adapter stays addressable through the rewritten tables, slots stay runs of
    consecutive cells."""
    from valora_b200.pool import AdapterPool
    width, n_slots = 128, 2
    pool = AdapterPool(cells=2 * (16 + 8 + 16 + 8), width=width, n_slots=n_slots, dtype=torch.float16, device=DEV)
    g = torch.Generator().manual_seed(3)
    blocks = {}
    for name, r in (("a", 16), ("b", 8), ("c", 16), ("d", 8)):
        blocks[name] = [torch.randn(r, width, generator=g).half() + 1.0 for _ in range(n_slots)]
        pool.load_adapter(name, r, 1.0, [blocks[name]])
    assert pool.can_use_mem_size == 0
    pool.offload_adapters(["b", "d"])                       # frees two separate runs of 32 cells
    # (1) a new adapter with an untouched projection lands on a's old cells
    blocks["e"] = [torch.randn(16, width, generator=g).half(), None]
    i = pool.load_adapter("e", 16, 1.0, [blocks["e"]])
    loc = pool.a_loc[pool.a_start[i]: pool.a_start[i] + 32]
    assert torch.equal(pool.buffer[0][loc[:16]].cpu(), blocks["e"][0])
    assert torch.count_nonzero(pool.buffer[0][loc[16:]]).item() == 0
    # (2) 32 cells are free, but as two runs of... make it so: drop e, load two rank-4 adapters
    pool.offload_adapters(["b", "d"])
    for name in ("f", "h"):
        blocks[name] = [torch.randn(4, width, generator=g).half() for _ in range(n_slots)]
        pool.load_adapter(name, 4, 1.0, [blocks[name]])     # 8 cells each, at the front of a's old run
    pool.offload_adapters(["b", "d", "h"])                  # free: 8 + 16 cells in a's run, 32 in c's run
    blocks["big"] = [torch.randn(24, width, generator=g).half() for _ in range(n_slots)]
    assert pool.can_use_mem_size == 56 and pool.alloc_contiguous(48) is None
    i = pool.load_adapter("big", 24, 1.0, [blocks["big"]])  # needs 48 consecutive cells: only after compaction
    assert pool.names == ["b", "d", "h", "big"]
    for k, name in enumerate(pool.names):
        r = blocks[name][0].shape[0]
        loc = pool.a_loc[pool.a_start[k]: pool.a_start[k] + n_slots * r].cpu()
        assert torch.equal(loc, torch.arange(int(loc[0]), int(loc[0]) + n_slots * r))
        for p in range(n_slots):
            assert torch.equal(pool.buffer[0][loc[p * r:(p + 1) * r].to(DEV)].cpu(), blocks[name][p]), (name, p)
    assert pool.can_use_mem_size == 8


def test_dropin_modules(ops):
    from valora_b200 import dropin
    dropin.install(force=True)
    from atmm_ops import dispatch_bgmv as dispatch_sgmm
    from valora._kernels import dispatch_bgmv
    H, ranks, N = 512, [16], 8
    A, B = rand_lora(ranks, H, H, torch.float16, n_slots=4, seed=1, wstd=0.1)
    a_start, a_len, a_loc, total = build_tables(ranks, 4)
    wa = fill_pool_a(A, ranks, a_start, a_loc, total, H, torch.float16)
    x = torch.randn(N, H).half()
    idx = torch.zeros(N, dtype=torch.int64)
    sc = torch.ones(1).half()
    ref = oracle.bgmv_shrink_ref(torch.zeros(N, 16).half(), x, wa, a_start, a_len, a_loc, idx, 1)
    v = torch.zeros(N, 16, dtype=torch.float16, device=DEV)
    dispatch_bgmv(v, x.to(DEV), wa.view(total, 8, 64).to(DEV), t64(a_start, DEV), t64(a_len, DEV),
                  t64(a_loc, DEV), idx.to(DEV), 1, sc.to(DEV))
    assert _err(v, ref) <= TOL
    v2 = torch.zeros(N, 16, dtype=torch.float16, device=DEV)
    dispatch_sgmm(v2, x.to(DEV), wa.view(total, 8, 64).to(DEV), t64(a_start, DEV), t64(a_len, DEV),
                  t64(a_loc, DEV), idx.to(DEV), 1, sc.to(DEV), t64([N], DEV), t64([16], DEV), t64([0], DEV),
                  t64([0, N], DEV), torch.zeros(60, dtype=torch.int8, device=DEV), 1, 64, 32, 32, 32, 32, 32)
    assert _err(v2, ref) <= TOL


def test_dropin_replays_a_layer_of_the_callers_sequence(ops):
    """The operator calls of one layer in the order the reference's caller issues them
    (lora_unordered_batch_infer.py:946-988 for q/k/v, :1611-1622 for o): three shrinks
    into zeroed [T, max_r] buffers (slots 0..2), three expands into q / k / v, then
    shrink + expand of slot 3 on the attention output - through the installed module
    names, with the problem table coming from the device packer instead of
    set_sgmm_args.  Reference semantics: no adapter scale in the ATMM expand."""
    from valora_b200 import dropin
    dropin.install(force=True)
    from atmm_ops import dispatch_bgmv as dispatch_sgmm
    dtype, H = torch.float16, 512
    ranks = [16, 64, 32]
    req_ad = [1, 0, 2, 1, 1, 0]
    req_len = [70, 130, 1, 1, 45, 9]
    tok = np.repeat(req_ad, req_len).astype(np.int64)
    T, max_r = tok.shape[0], max(ranks)
    A, B = rand_lora(ranks, H, H, dtype, n_slots=4, seed=21, wstd=0.05)
    a_start, a_len, a_loc, total = build_tables(ranks, 4, shuffle=True, contiguous_slots=True, seed=3)
    key_buffer = fill_pool_a(A, ranks, a_start, a_loc, total, H, dtype).view(total, 8, H // 8).to(DEV)
    value_buffer = fill_pool_b(B, ranks, a_start, a_loc, total, H, dtype, layout="rows").view(total, 8, H // 8).to(DEV)
    ast_d, alen_d, aloc_d = t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV)
    scaling = torch.ones(len(ranks), dtype=dtype, device=DEV)
    # the batch's problem table, in request order (the reference's run-length encoding)
    packer = ops.Packer(T, len(ranks), DEV)
    pk = packer.pack(torch.from_numpy(tok).to(DEV), alen_d, sort=False)
    P = pk.host_counts()["P"]
    tables = (pk.seg_len, pk.seg_rank, pk.seg_adapter, pk.seg_start)
    tmp_d = torch.zeros(60 * 128, dtype=torch.int8, device=DEV)
    tiles = (64, 32, 32, 32, 32, 32)
    bins = torch.from_numpy(tok).to(DEV)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, H, generator=g).to(dtype)
    outs0 = [torch.randn(T, H, generator=g).to(dtype) for _ in range(4)]        # q, k, v, o before LoRA
    attn = torch.randn(T, H, generator=g).to(dtype)                             # input of the o projection
    delta = [torch.zeros(T, max_r, dtype=dtype, device=DEV) for _ in range(4)]
    outs = [o.to(DEV) for o in outs0]
    xd, attnd = x.to(DEV), attn.to(DEV)
    for slot in range(3):
        dispatch_sgmm(delta[slot], xd, key_buffer, ast_d, alen_d, aloc_d, bins, slot, scaling, *tables, tmp_d, P, *tiles)
    torch.cuda.synchronize()
    for slot in range(3):
        dispatch_sgmm(outs[slot], delta[slot], value_buffer, ast_d, alen_d, aloc_d, bins, slot, scaling, *tables,
                      tmp_d, P, *tiles)
    torch.cuda.synchronize()
    dispatch_sgmm(delta[3], attnd, key_buffer, ast_d, alen_d, aloc_d, bins, 3, scaling, *tables, tmp_d, P, *tiles)
    dispatch_sgmm(outs[3], delta[3], value_buffer, ast_d, alen_d, aloc_d, bins, 3, scaling, *tables, tmp_d, P, *tiles)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    oc, rc, li, si = (v[:P + (1 if i == 3 else 0)].cpu().numpy() for i, v in enumerate(tables))
    wa, wb = key_buffer.cpu().view(total, H), value_buffer.cpu().view(total, H)
    for slot in range(4):
        src = attn if slot == 3 else x
        v_ref = oracle.atmm_shrink_ref(torch.zeros(T, max_r, dtype=dtype), src, wa, a_start, a_loc, slot, oc, rc, li, si, P)
        assert _err(delta[slot], v_ref) <= TOL
        y_ref = oracle.atmm_expand_ref(outs0[slot], v_ref.to(dtype), wb, a_start, a_loc, slot, oc, rc, li, si, P)
        assert _err(outs[slot], y_ref) <= TOL


def test_dropin_replays_the_merged_adapter_correction(ops):
    """One adapter is folded into the base weight (merged mode) while requests of other
    adapters share the batch.  The caller's correction (lora_unordered_batch_infer.py:
    991-1063): the rows after the merged adapter's are stacked twice, the first copy runs
    with each row's own adapter, the second with the merged adapter, and
    `q[tk:] += out[:L] - out[L:]` takes the merged contribution out again.  Replayed
    through the installed module name; the end result must be base + own adapter."""
    from valora_b200 import dropin
    dropin.install(force=True)
    from atmm_ops import dispatch_bgmv as dispatch_sgmm
    dtype, H = torch.float16, 512
    ranks = [32, 16, 64, 16]
    merged = 2
    req_ad = [2, 2, 0, 1, 3, 0, 1, 1]                       # the merged adapter's requests lead the batch
    req_len = [40, 1, 90, 1, 1, 33, 1, 150]
    tok = np.repeat(req_ad, req_len).astype(np.int64)
    T, max_r = tok.shape[0], max(ranks)
    tk = int(sum(l for a, l in zip(req_ad, req_len) if a == merged))
    L = T - tk
    A, B = rand_lora(ranks, H, H, dtype, n_slots=4, seed=31, wstd=0.05)
    a_start, a_len, a_loc, total = build_tables(ranks, 4, shuffle=True, contiguous_slots=True, seed=4)
    key_buffer = fill_pool_a(A, ranks, a_start, a_loc, total, H, dtype).view(total, 8, H // 8).to(DEV)
    value_buffer = fill_pool_b(B, ranks, a_start, a_loc, total, H, dtype, layout="rows").view(total, 8, H // 8).to(DEV)
    ast_d, alen_d, aloc_d = t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV)
    scaling = torch.ones(len(ranks), dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(6)
    x = torch.randn(T, H, generator=g).to(dtype)
    slot = 1
    W0 = (torch.randn(H, H, generator=g) * 0.02).to(dtype)
    Wm = (W0.float() + A[slot][merged].float() @ B[slot][merged].float()).to(dtype)     # merged mode, scale 1
    q0 = (x.float() @ Wm.float()).to(dtype)                                              # base projection
    # problem table of the stacked rows: own adapters over [0, L), the merged one over [L, 2L)
    tok2 = np.concatenate([tok[tk:], np.full(L, merged, np.int64)])
    packer = ops.Packer(2 * L, len(ranks), DEV)
    pk = packer.pack(torch.from_numpy(tok2).to(DEV), alen_d, sort=False)
    P = pk.host_counts()["P"]
    tables = (pk.seg_len, pk.seg_rank, pk.seg_adapter, pk.seg_start)
    tmp_d = torch.zeros(60 * 128, dtype=torch.int8, device=DEV)
    tiles = (64, 32, 32, 32, 32, 32)
    bins = torch.from_numpy(tok2).to(DEV)
    q = q0.to(DEV)
    sub = x.to(DEV)[tk:]
    stacked = torch.cat([sub, sub], dim=0)
    delta = torch.zeros(2 * L, max_r, dtype=dtype, device=DEV)
    out = torch.zeros(2 * L, H, dtype=dtype, device=DEV)
    dispatch_sgmm(delta, stacked, key_buffer, ast_d, alen_d, aloc_d, bins, slot, scaling, *tables, tmp_d, P, *tiles)
    torch.cuda.synchronize()
    dispatch_sgmm(out, delta, value_buffer, ast_d, alen_d, aloc_d, bins, slot, scaling, *tables, tmp_d, P, *tiles)
    q[tk:] += out[:L] - out[L:]
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    # each half against the restated operator, then the end result against base + own adapter in fp32
    oc, rc, li, si = (v[:P + (1 if i == 3 else 0)].cpu().numpy() for i, v in enumerate(tables))
    wa, wb = key_buffer.cpu().view(total, H), value_buffer.cpu().view(total, H)
    v_ref = oracle.atmm_shrink_ref(torch.zeros(2 * L, max_r, dtype=dtype), stacked.cpu(), wa, a_start, a_loc, slot,
                                   oc, rc, li, si, P)
    assert _err(delta, v_ref) <= TOL
    o_ref = oracle.atmm_expand_ref(torch.zeros(2 * L, H, dtype=dtype), v_ref.to(dtype), wb, a_start, a_loc, slot,
                                   oc, rc, li, si, P)
    assert _err(out, o_ref) <= TOL
    want = x.float() @ W0.float()
    for t in range(T):
        a = int(tok[t])
        want[t] += (x[t].float() @ A[slot][a].float()) @ B[slot][a].float()
    assert torch.equal(q[:tk].cpu(), q0[:tk])                               # the merged adapter's rows are not touched
    assert (q.cpu().float() - want).abs().max().item() <= 2e-2              # three roundings of a 16-bit q on the way


# --------------------------------------------------------------------------- step (packed batch, many problems)
def _step_case(ops, batch, proj_ids, layers=1, mma_min=16, gather_path="mma", wide_gather=None):
    from valora_b200.engine import LoraStepEngine
    projs = [batch.projections[p] for p in proj_ids]
    eng = LoraStepEngine(projs, batch.ranks, batch.scalings(), batch.dtype, DEV, layers, batch.T,
                         mma_min_rows=mma_min, gather_path=gather_path, wide_gather=wide_gather)
    g = torch.Generator().manual_seed(batch.seed)
    W = {}
    for layer in range(layers):
        for p, (_, hi, ho) in enumerate(projs):
            for a in range(batch.n_adapters):
                r = int(batch.ranks[a])
                A = (torch.randn(hi, r, generator=g) * 0.02).to(batch.dtype)
                B = (torch.randn(r, ho, generator=g) * 0.02).to(batch.dtype)
                W[(layer, p, a)] = (A, B)
                eng.set_adapter_weights(layer, p, a, A, B)
    X, Y0 = {}, {}
    for layer in range(layers):
        for p, (_, hi, ho) in enumerate(projs):
            X[(layer, p)] = torch.randn(batch.T, hi, generator=g).to(batch.dtype)
            Y0[(layer, p)] = torch.randn(batch.T, ho, generator=g).to(batch.dtype)
            eng.x[layer][p].copy_(X[(layer, p)])
            eng.y[layer][p].copy_(Y0[(layer, p)])
    tok = torch.from_numpy(batch.tok_adapter.astype(np.int64)).to(DEV)
    eng.step(tok)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    sc = batch.scalings()
    worst_own = 0.0
    for layer in range(layers):
        for p in range(len(projs)):
            truth = Y0[(layer, p)].float().clone()
            xf = X[(layer, p)].float()
            for a in np.unique(batch.tok_adapter):
                rows = torch.from_numpy(np.nonzero(batch.tok_adapter == a)[0])
                A, B = W[(layer, p, int(a))]
                # the operator's fp32 truth: nothing is rounded before the result (the kernels
                # keep V in a 16-bit buffer between shrink and expand, as the reference does;
                # that rounding is part of the error measured here)
                truth[rows] += ((xf[rows] @ A.float()) @ B.float()) * float(sc[a])
            assert _err(eng.y[layer][p], truth) <= TOL, (layer, p)
            own = own_error(eng.y[layer][p], truth)
            worst_own = max(worst_own, own)
            assert own <= OWN_TOL, (layer, p, own)
    print(f"step {batch.name} projections {proj_ids}: kernels' own error (output half-ulp taken off) {worst_own:.3e}")
    return eng


@pytest.mark.parametrize("gather_path", ["mma", "simt"])
def test_step_config0(ops, gather_path):
    _step_case(ops, workloads.config0(), [0], gather_path=gather_path)


@pytest.mark.parametrize("gather_path", ["mma", "simt"])
def test_step_config3_mixed_two_widths(ops, gather_path):
    """mixed prefill + decode batch of config 3, one layer, q / up / down projections
    (4096->4096, 4096->11008, 11008->4096): consecutive-row tiles and gathered rows together"""
    _step_case(ops, workloads.config3(layers=1), [0, 4, 6], gather_path=gather_path)


def test_step_config2_hetero_ranks_two_layers(ops):
    b = workloads.config2()
    _step_case(ops, b, [0, 3], layers=2)


def test_step_config2_all_seven_projections(ops):
    """config 2 whole: fp16, ranks 8..128, all seven projection shapes of one layer"""
    _step_case(ops, workloads.config2(), list(range(7)))


def test_step_config3_all_seven_projections_two_layers(ops):
    """the benchmarked batch (config 3) on all seven projection shapes, two layers: the
    problem mix of the timed launch at 1/16 of its depth"""
    _step_case(ops, workloads.config3(layers=2), list(range(7)), layers=2)


def test_step_config4_whole_single_gpu(ops):
    """config 4 as one GPU sees it alone: 16384 tokens, 1024 adapters of ranks 16..128,
    25 % prefill rows and 75 % decode rows, every row against the fp32 truth"""
    b = workloads.config4()
    assert b.T == 16384 and b.n_adapters == 1024
    _step_case(ops, b, [0])


@pytest.mark.parametrize("gather_path", ["mma", "simt"])
def test_step_all_gather_rows(ops, gather_path):
    """decode-only batch (config 1): every row is a gathered row"""
    _step_case(ops, workloads.config1(), [0], gather_path=gather_path)


@pytest.mark.parametrize("overlap", [False, True])
def test_step_from_host_buffers_matches_resident_step(ops, overlap):
    """step_host (pinned host buffers in, Y out, optionally pipelined by layer over
    three streams) gives bit for bit what step() gives on resident inputs, twice in
    a row (the second call re-uses the device buffers the first one wrote)."""
    from valora_b200.engine import LoraStepEngine
    b = workloads.config0()
    if overlap:
        # ranks on both sides of 64: every layer's call forks and joins the side stream of the tile classes
        b.ranks = np.array([8, 128, 16, 72], np.int64)
    projs = [("q", 512, 512), ("up", 512, 1024)]
    L = 3
    eng = LoraStepEngine(projs, b.ranks, b.scalings(), b.dtype, DEV, L, b.T)
    assert bool(eng._gather_flag() & ops.STEP_SPLIT_RANK_CLASSES) == bool(overlap)
    eng.randomize_weights(seed=5)
    g = torch.Generator().manual_seed(9)
    xh = [[torch.randn(b.T, hi, generator=g).to(b.dtype).pin_memory() for _, hi, _ in projs] for _ in range(L)]
    yh = [[torch.randn(b.T, ho, generator=g).to(b.dtype).pin_memory() for _, _, ho in projs] for _ in range(L)]
    out = [[torch.zeros(b.T, ho, dtype=b.dtype).pin_memory() for _, _, ho in projs] for _ in range(L)]
    tok_h = torch.from_numpy(b.tok_adapter.astype(np.int64)).pin_memory()
    tok_d = torch.empty(b.T, dtype=torch.int64, device=DEV)
    # resident reference
    for l in range(L):
        for p in range(len(projs)):
            eng.x[l][p].copy_(xh[l][p])
            eng.y[l][p].copy_(yh[l][p])
    eng.step(tok_h.to(DEV))
    torch.cuda.synchronize()
    want = [[eng.y[l][p].cpu() for p in range(len(projs))] for l in range(L)]
    for _ in range(2):
        h2d, d2h = eng.step_host(tok_h, xh, yh, tok_d, y_out_host=out, overlap=overlap)
        torch.cuda.current_stream().synchronize()
        assert ops.device_status() == 0
        for l in range(L):
            for p in range(len(projs)):
                assert torch.equal(out[l][p], want[l][p]), (l, p)
                out[l][p].zero_()
    assert h2d == b.T * 8 + L * b.T * (512 + 512 + 512 + 1024) * 2 and d2h == L * b.T * (512 + 1024) * 2


def test_step_shared_inputs_match_private_copies(ops):
    """q/k/v-style groups: three projections that read ONE activation buffer give bit for
    bit what three private copies of it give, resident and from host buffers (where the
    shared X crosses the link once)."""
    from valora_b200.engine import LoraStepEngine
    b = workloads.config0()
    projs = [("q", 512, 512), ("k", 512, 256), ("v", 512, 256), ("o", 512, 512), ("up", 512, 1024), ("gate", 512, 1024)]
    input_of = [0, 0, 0, 3, 4, 4]
    L = 2
    shared = LoraStepEngine(projs, b.ranks, b.scalings(), b.dtype, DEV, L, b.T, input_of=input_of)
    private = LoraStepEngine(projs, b.ranks, b.scalings(), b.dtype, DEV, L, b.T)
    shared.randomize_weights(seed=6)
    private.randomize_weights(seed=6)
    assert shared.x[0][1] is shared.x[0][0] and shared.x[1][5] is shared.x[1][4] and shared.x[0][3] is not shared.x[0][0]
    g = torch.Generator().manual_seed(10)
    xh = [[torch.randn(b.T, hi, generator=g).to(b.dtype).pin_memory() for _, hi, _ in projs] for _ in range(L)]
    yh = [[torch.randn(b.T, ho, generator=g).to(b.dtype).pin_memory() for _, _, ho in projs] for _ in range(L)]
    for l in range(L):
        for p in range(len(projs)):
            private.x[l][p].copy_(xh[l][input_of[p]])
            private.y[l][p].copy_(yh[l][p])
            shared.y[l][p].copy_(yh[l][p])
            if input_of[p] == p:
                shared.x[l][p].copy_(xh[l][p])
    tok = torch.from_numpy(b.tok_adapter.astype(np.int64)).to(DEV)
    private.step(tok)
    shared.step(tok)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for l in range(L):
        for p in range(len(projs)):
            assert torch.equal(shared.y[l][p], private.y[l][p]), (l, p)
    # oracle on one problem of a group
    A, B = zip(*[private.adapter_weights(1, 2, a) for a in range(len(b.ranks))])
    want = oracle.ragged_lora_ref_fp32(yh[1][2], xh[1][0], [a.cpu() for a in A], [bb.cpu() for bb in B],
                                  b.req_len, b.req_adapter, b.scalings())
    assert (shared.y[1][2].cpu().float() - want).abs().max().item() <= 1e-2
    # from host buffers: entries of xh that are not a group's first are never read
    out = [[torch.zeros(b.T, ho, dtype=b.dtype).pin_memory() for _, _, ho in projs] for _ in range(L)]
    tok_h = torch.from_numpy(b.tok_adapter.astype(np.int64)).pin_memory()
    tok_d = torch.empty(b.T, dtype=torch.int64, device=DEV)
    h2d, d2h = shared.step_host(tok_h, xh, yh, tok_d, y_out_host=out)
    torch.cuda.current_stream().synchronize()
    for l in range(L):
        for p in range(len(projs)):
            assert torch.equal(out[l][p], private.y[l][p].cpu()), (l, p)
    assert h2d == b.T * 8 + L * b.T * (3 * 512 + sum(ho for _, _, ho in projs)) * 2
    with pytest.raises(ValueError):
        LoraStepEngine(projs, b.ranks, b.scalings(), b.dtype, DEV, 1, b.T, input_of=[0, 0, 1, 3, 4, 4])
    with pytest.raises(ValueError):
        LoraStepEngine([("a", 512, 512), ("b", 256, 512)], b.ranks, b.scalings(), b.dtype, DEV, 1, b.T, input_of=[0, 0])


@pytest.mark.parametrize("mixed_ranks", [False, True])
def test_step_replays_from_a_cuda_graph(ops, mixed_ranks):
    """packer + shrink + expand captured once, replayed on batches whose token -> adapter
    map changes between replays: the schedule is rebuilt on the device inside the graph,
    so every replay must equal an eager step on the same inputs, bit for bit.  With ranks
    above 64 in the pool the step forks a side stream for one class of tiles and joins it
    again: that too has to sit inside the captured graph."""
    from valora_b200.engine import LoraStepEngine
    b = workloads.config3(layers=1)
    if mixed_ranks:
        b.ranks = np.random.default_rng(6).choice(np.array([16, 64, 128]), size=b.n_adapters).astype(np.int64)
    projs = [("q", 1024, 1024), ("up", 1024, 2048)]
    L = 2
    eng = LoraStepEngine(projs, b.ranks, b.scalings(), b.dtype, DEV, L, b.T)
    assert bool(eng._gather_flag() & ops.STEP_SPLIT_RANK_CLASSES) == mixed_ranks
    eng.randomize_weights(seed=12)
    g = torch.Generator(device=DEV)
    g.manual_seed(13)
    x0 = [[torch.randn(b.T, hi, generator=g, device=DEV).to(b.dtype) for _, hi, _ in projs] for _ in range(L)]
    y0 = [[torch.randn(b.T, ho, generator=g, device=DEV).to(b.dtype) for _, _, ho in projs] for _ in range(L)]

    def reset():
        for l in range(L):
            for p in range(len(projs)):
                eng.x[l][p].copy_(x0[l][p])
                eng.y[l][p].copy_(y0[l][p])

    rng = np.random.default_rng(5)
    toks = [b.tok_adapter.astype(np.int64)]
    toks.append(np.roll(toks[0], 777))                                   # other rows become the decode rows
    toks.append(rng.integers(0, b.n_adapters, size=b.T).astype(np.int64))  # no consecutive runs at all
    tok_buf = torch.from_numpy(toks[0]).to(DEV)
    eager = []
    for t in toks:
        reset()
        tok_buf.copy_(torch.from_numpy(t))
        eng.step(tok_buf)
        torch.cuda.synchronize()
        eager.append([[eng.y[l][p].clone() for p in range(len(projs))] for l in range(L)])
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        eng.step(tok_buf)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        eng.step(tok_buf)
    for i in (2, 0, 1, 1):
        reset()
        tok_buf.copy_(torch.from_numpy(toks[i]))
        graph.replay()
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        for l in range(L):
            for p in range(len(projs)):
                assert torch.equal(eng.y[l][p], eager[i][l][p]), (i, l, p)


@pytest.mark.parametrize("gather_path", ["mma", "simt"])
def test_step_narrow_projections(ops, gather_path):
    """projections narrower than the 128-wide rank buffer (64 -> 64, 64 -> 192, 128 -> 64):
    the step must still run shrink as shrink and expand as expand"""
    b = workloads.config0()
    b.projections = [("a", 64, 64), ("b", 64, 192), ("c", 128, 64)]
    _step_case(ops, b, [0, 1, 2], layers=2, gather_path=gather_path)


@pytest.mark.parametrize("wide", [False, True])
def test_step_gather_stage_forms(ops, wide):
    """both forms of the expand's gather stages (at most four 64-column blocks / as many as fit)
    on both kinds of batch: rank 64 everywhere (config 3, 4096 -> 11008) and ranks 16..128 with
    mostly decode rows (config 4 slice)"""
    _step_case(ops, workloads.config3(layers=1), [4], wide_gather=wide)
    _step_case(ops, workloads.config4(n_gpus=8, rank=5), [0], wide_gather=wide)


def test_step_gathered_rows_mixed_ranks(ops):
    """config 4 slice: 1024 adapters of ranks 16..128, mostly decode rows, many adapters
    with a handful of rows each - gathered tiles of every rank on the tensor cores"""
    b = workloads.config4(n_gpus=8, rank=3)
    _step_case(ops, b, [0])


# --------------------------------------------------------------------------- merged mode
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_merge_and_unmerge_adapter(ops, dtype):
    """W +- scaling * A @ B on the expand kernel (rows of W as tokens), against fp32 torch;
    merge followed by unmerge returns W up to the two roundings."""
    from valora_b200 import merge
    from valora_b200.pool import AdapterPool
    h_in, h_out, ranks = 1024, 1536, [16, 64, 24]
    pa = AdapterPool(sum(ranks) * 2 + 16, h_in, 2, dtype, DEV, 1)
    pb = AdapterPool(sum(ranks) * 2 + 16, h_out, 2, dtype, DEV, 1)
    g = torch.Generator().manual_seed(4)
    A, B = {}, {}
    for a, r in enumerate(ranks):
        A[a] = [(torch.randn(r, h_in, generator=g) * 0.05).to(dtype) for _ in range(2)]     # A^T rows per slot
        B[a] = [(torch.randn(r, h_out, generator=g) * 0.05).to(dtype) for _ in range(2)]
        pa.load_adapter(f"a{a}", r, 16.0 / r, [[A[a][0], A[a][1]]])
        pb.load_adapter(f"a{a}", r, 16.0 / r, [[B[a][0], B[a][1]]])
    W0 = torch.randn(h_in, h_out, generator=g).to(dtype)
    for adapter, slot in ((1, 0), (2, 1), (0, 1)):
        W = W0.to(DEV)
        merge.merge_adapter(W, pa, pb, 0, slot, slot, adapter)
        s = float(torch.tensor(16.0 / ranks[adapter]).to(dtype))
        want = W0.float() + s * (A[adapter][slot].float().t() @ B[adapter][slot].float())
        assert _err(W, want) <= TOL
        merge.unmerge_adapter(W, pa, pb, 0, slot, slot, adapter)
        assert float((W.float().cpu() - W0.float()).abs().max()) <= 4e-2                      # two roundings of |w| < 8
    assert ops.device_status() == 0


# --------------------------------------------------------------------------- device status and bounded waits
def test_bounded_wait_gives_up_and_reports(ops):
    """A wait that nothing will ever complete (a freshly initialised barrier nobody arrives
    on) runs out of its small cycle budget, the kernel returns normally and raises status
    bit 1 - in the caller's own status word, and in the process-wide one when none is given.
    Nothing faults: the next kernel on the same context runs as usual."""
    assert ops.device_status() == 0
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    waited = ops.selftest_bounded_wait(200_000, DEV, status=word)
    assert int(word.item()) == 1
    assert 200_000 <= waited < 50_000_000                   # gave up after the budget, not after the 1 s default
    assert ops.device_status(reset=False) == 0               # the process-wide word was not touched
    ops.selftest_bounded_wait(50_000, DEV)
    assert ops.device_status() == 1                          # read and cleared
    assert ops.device_status() == 0
    # the context is alive: a real kernel right after
    v = torch.zeros(4, 16, dtype=torch.float16, device=DEV)
    x = torch.ones(4, 256, dtype=torch.float16, device=DEV)
    w = torch.ones(32, 1, 256, dtype=torch.float16, device=DEV)
    z = torch.zeros(1, dtype=torch.int64, device=DEV)
    ops.bgmv(v, x, w, z, torch.full((1,), 64, dtype=torch.int64, device=DEV), torch.arange(16, device=DEV),
             torch.zeros(4, dtype=torch.int64, device=DEV), 0, torch.ones(1, dtype=torch.float16, device=DEV))
    assert torch.all(v.cpu() == 256.0)


def test_step_reports_skipped_tiles_in_its_own_status_word(ops):
    """A step told that no adapter exceeds rank 16 skips the tiles of a rank-64 adapter and
    says so (status bit 2) in the status word it was given; with the true bound the same
    step is clean.  Rows of skipped tiles keep their input."""
    from valora_b200.engine import LoraStepEngine
    ranks = np.array([16, 64])
    tok = np.repeat([0, 1], [40, 24]).astype(np.int64)
    eng = LoraStepEngine([("p", 256, 256)], ranks, (16.0 / ranks).astype(np.float32), torch.float16, DEV, 1, 64)
    eng.randomize_weights(seed=2)
    eng.x[0][0].normal_()
    y0 = torch.randn(64, 256, device=DEV).half()
    eng.y[0][0].copy_(y0)
    packed = eng.packer.pack(torch.from_numpy(tok).to(DEV), eng.a_len)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    flags = ops.PHASE_ALL | eng._gather_flag()
    eng.plan.run(packed, eng.scales, phase_mask=flags, max_rank=16, status=word)
    torch.cuda.synchronize()
    assert int(word.item()) == 2
    assert torch.equal(eng.y[0][0][40:], y0[40:]) and not torch.equal(eng.y[0][0][:40], y0[:40])
    assert ops.device_status() == 0                          # the process-wide word stays clean
    word.zero_()
    eng.plan.run(packed, eng.scales, phase_mask=flags, max_rank=64, status=word)
    torch.cuda.synchronize()
    assert int(word.item()) == 0
    with pytest.raises(RuntimeError):
        ops.Packer(64, 2, DEV, tile_m=256)                   # a tile is one MMA tile at most
    with pytest.raises(RuntimeError):
        ops.Packer(64, 2, DEV, gather_rows_per_tile=64)


# --------------------------------------------------------------------------- base projection with the expand folded in
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_projection_matches_base_plus_lora(ops, dtype):
    """y = x W + s (x A) B in one pass over y (written, never read) for the rows of the
    consecutive-row tiles; rows of gather tiles keep what they held.  Checked against
    fp32 torch on the same V' (the kernel's arithmetic) and against the operator's fp32
    truth with nothing rounded on the way (V' is a 16-bit tensor, scaled before its one
    rounding by the shrink's apply_scale)."""
    h_in, h_out = 512, 768
    ranks = [8, 16, 64, 128, 32]
    seg_len = [300, 129, 5, 64, 17, 200, 3]
    seg_ad = [1, 0, 4, 2, 1, 3, 0]
    tok = np.repeat(seg_ad, seg_len).astype(np.int64)
    T = tok.shape[0]
    A, B = rand_lora(ranks, h_in, h_out, dtype, n_slots=2, seed=51, wstd=0.02)
    a_start, a_len, a_loc, total = build_tables(ranks, 2, shuffle=True, contiguous_slots=True, seed=52)
    slot = 1
    wa = fill_pool_a(A, ranks, a_start, a_loc, total, h_in, dtype)
    wb = fill_pool_b(B, ranks, a_start, a_loc, total, h_out, dtype, layout="rows")
    g = torch.Generator().manual_seed(53)
    x = torch.randn(T, h_in, generator=g).to(dtype)
    W = (torch.randn(h_in, h_out, generator=g) * 0.05).to(dtype)
    scales = torch.tensor([16.0 / r for r in ranks]).to(dtype)
    dev = lambda t: t.to(DEV)
    packer = ops.Packer(T, len(ranks), DEV)
    alen_d = t64(a_len, DEV)
    # V' from the shrink entry point with the scale applied (problem table in batch order)
    pk0 = packer.pack(torch.from_numpy(tok).to(DEV), alen_d, sort=False)
    P = pk0.host_counts()["P"]
    vp = torch.zeros(T, 128, dtype=dtype, device=DEV)
    ops.atmm(vp, dev(x), dev(wa).view(total, 1, h_in), t64(a_start, DEV), alen_d, t64(a_loc, DEV),
             torch.from_numpy(tok).to(DEV), slot, dev(scales), pk0.seg_len.clone(), pk0.seg_rank.clone(),
             pk0.seg_adapter.clone(), pk0.seg_start.clone(), None, P, apply_scale=True)
    torch.cuda.synchronize()
    v_truth = torch.zeros(T, 128)
    for t in range(T):
        a = int(tok[t])
        v_truth[t, :ranks[a]] = (x[t].float() @ A[slot][a].float()) * float(scales[a])
    assert _err(vp, v_truth) <= TOL
    # the fused projection on the sorted schedule
    pk = packer.pack(torch.from_numpy(tok).to(DEV), alen_d, sort=True)
    c = pk.host_counts()
    assert c["n_mma"] > 0 and c["n_gather"] > 0
    y = torch.full((T, h_out), float("nan"), dtype=dtype, device=DEV)
    ops.fused_proj(y, dev(x), dev(W), vp, dev(wb), t64(a_start, DEV), t64(a_loc, DEV), slot, pk)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    in_gather = np.isin(tok, [4]) | (np.arange(T) >= T - 3)          # the 5-row and the 3-row run
    yc = y.cpu()
    assert torch.isnan(yc[torch.from_numpy(in_gather)].float()).all()     # untouched
    rows = torch.from_numpy(~in_gather)
    same_v = x.float() @ W.float()
    truth = same_v.clone()
    vpc = vp.cpu().float()
    for t in range(T):
        a = int(tok[t])
        same_v[t] += vpc[t, :ranks[a]] @ B[slot][a].float()
        truth[t] += ((x[t].float() @ A[slot][a].float()) @ B[slot][a].float()) * float(scales[a])
    assert _err(y[dev(rows)], same_v[rows]) <= TOL
    assert own_error(y[dev(rows)], same_v[rows]) <= 1e-4            # fp32 accumulation order only
    assert _err(y[dev(rows)], truth[rows]) <= TOL
    assert own_error(y[dev(rows)], truth[rows]) <= OWN_TOL


def test_results_do_not_depend_on_the_tile_table(ops):
    """The tile table changes how a launch is cut into stages and tiles, never what it
    computes: a drop-in shrink + expand and a step give bit-identical results under every
    choice the table may hold (ring of 2 / 3 / 4 stages, small-call tiles of 32 / 64 / 128 rows,
    wide gather stages for no / some / all adapters)."""
    import json
    from valora_b200 import _lib, tile_table
    from valora_b200.engine import LoraStepEngine
    lib = _lib.load()
    base = tile_table.load(tile_table.DEFAULT_PATH)

    def table(ss, es, rows, wide):
        t = json.loads(json.dumps(base))
        for e in t["entries"]:
            e.update(shrink_stages=min(ss, 3) if e["max_rank"] > 64 else ss, expand_stages=3 if e["max_rank"] > 64 else es,
                     small_call_rows=rows, wide_gather_below_rank=wide)
        return t

    dtype, h = torch.bfloat16, 1024
    ranks = [16, 64, 8, 32]
    seg_len, seg_ad = [5, 140, 33, 1, 70], [0, 1, 2, 3, 1]
    A, B = rand_lora(ranks, h, h, dtype, n_slots=1, seed=61)
    a_start, a_len, a_loc, total = build_tables(ranks, 1, shuffle=True, contiguous_slots=True, seed=62)
    wa = fill_pool_a(A, ranks, a_start, a_loc, total, h, dtype).to(DEV)
    wb = fill_pool_b(B, ranks, a_start, a_loc, total, h, dtype, layout="rows").to(DEV)
    T = sum(seg_len)
    g = torch.Generator().manual_seed(63)
    x = torch.randn(T, h, generator=g).to(dtype).to(DEV)
    y0 = torch.randn(T, h, generator=g).to(dtype).to(DEV)
    oc, rc = t64(seg_len, DEV), t64([ranks[a] for a in seg_ad], DEV)
    li, si = t64(seg_ad, DEV), t64(np.concatenate([[0], np.cumsum(seg_len)]), DEV)
    idx = torch.zeros(T, dtype=torch.int64, device=DEV)
    sc = torch.tensor([16.0 / r for r in ranks]).to(dtype).to(DEV)
    tabs = (t64(a_start, DEV), t64(a_len, DEV), t64(a_loc, DEV))
    # a step on a decode-heavy batch with small and large ranks (gather tiles of both stage forms)
    b4 = workloads.config4(n_gpus=8, rank=2)
    outs = []
    try:
        for ss, es, rows, wide in ((4, 4, 32, 33), (3, 3, 64, 0), (2, 4, 128, 129)):
            tile_table.apply(lib, table(ss, es, rows, wide))
            v = torch.zeros(T, 64, dtype=dtype, device=DEV)
            ops.atmm(v, x, wa.view(total, 1, h), *tabs, idx, 0, sc, oc, rc, li, si, None, len(seg_len))
            y = y0.clone()
            ops.atmm(y, v, wb.view(total, 1, h), *tabs, idx, 0, sc, oc, rc, li, si, None, len(seg_len), apply_scale=True)
            eng = LoraStepEngine([("p", 512, 768)], b4.ranks, b4.scalings(), dtype, DEV, 1, b4.T)
            eng.randomize_weights(seed=64)
            gg = torch.Generator(device=DEV)
            gg.manual_seed(65)
            eng.x[0][0].normal_(generator=gg)
            eng.y[0][0].normal_(generator=gg)
            eng.step(torch.from_numpy(b4.tok_adapter.astype(np.int64)).to(DEV))
            torch.cuda.synchronize()
            assert ops.device_status() == 0
            outs.append((v.cpu(), y.cpu(), eng.y[0][0].cpu()))
            del eng
    finally:
        tile_table.apply(lib, base)
    for o in outs[1:]:
        for a, b in zip(outs[0], o):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_rank_class_split_changes_nothing(ops):
    """With an adapter above rank 64 resident a step launches each tensor-core kernel twice
    (VLR_STEP_SPLIT_RANK_CLASSES): once over the consecutive-row tiles above rank 64, once over
    all other tiles.  Every tile is taken by exactly one of the two launches: the results equal
    those of the single launch bit for bit."""
    from valora_b200.engine import LoraStepEngine
    dtype = torch.bfloat16
    b4 = workloads.config4(n_gpus=8, rank=5)
    assert min(b4.ranks) <= 64 < max(b4.ranks)
    tok = torch.from_numpy(b4.tok_adapter.astype(np.int64)).to(DEV)
    # second case: the only adapter above rank 64 is resident but not in the batch - the launches of
    # that class find no tile
    unused = sorted(set(range(len(b4.ranks))) - set(np.unique(b4.tok_adapter).tolist()))
    assert unused
    lone = np.minimum(b4.ranks, 64)
    lone[unused[0]] = 128
    # third case: every adapter at rank 128 - gather tiles on the four-stage ring, consecutive rows on three
    for ranks in (b4.ranks, lone, np.full_like(b4.ranks, 128)):
        scal = (workloads.ALPHA / ranks).astype(np.float32)
        outs = []
        for split in (True, False):
            eng = LoraStepEngine([("p", 1024, 512), ("q", 512, 1024)], ranks, scal, dtype, DEV, 2, b4.T,
                                 split_rank_classes=split)
            assert bool(eng._gather_flag() & ops.STEP_SPLIT_RANK_CLASSES) == split
            eng.randomize_weights(seed=71)
            gg = torch.Generator(device=DEV)
            gg.manual_seed(72)
            for l in range(2):
                for p in range(2):
                    eng.x[l][p].normal_(generator=gg)
                    eng.y[l][p].normal_(generator=gg)
            y0 = eng.y[1][1].clone()
            eng.step(tok)
            torch.cuda.synchronize()
            assert ops.device_status() == 0
            assert not torch.equal(y0, eng.y[1][1])
            outs.append([eng.y[l][p].cpu() for l in range(2) for p in range(2)])
            del eng
        for a, b in zip(*outs):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_step_random_ranks_widths_and_lengths(ops, seed):
    """Seeded random batches on the step: every rank the kernels take (multiples of 8 up to 128,
    so rank % 16 == 8 as well, on both sides of the rank-class split), widths whose K blocks do
    not fill the last stage of a gather tile (9, 13, 17 blocks), requests of 1 .. 200 tokens in
    random order, so that a segment mixes consecutive-row tiles, short chunks and single rows,
    and gather tiles of 1 .. 32 rows occur."""
    rng = np.random.default_rng(1000 + seed)
    n_ad = 24
    ranks = rng.choice(np.arange(8, 129, 8), size=n_ad).astype(np.int64)
    ranks[:4] = [8, 24, 72, 128]
    n_req = 90
    req_ad = rng.integers(0, n_ad, size=n_req).astype(np.int32)
    req_len = np.where(rng.random(n_req) < 0.7, 1, rng.integers(2, 200, size=n_req)).astype(np.int64)
    # a popular adapter with many decode rows: gather tiles of 32 rows and a remainder
    req_ad[:45] = np.where(rng.random(45) < 0.8, 3, req_ad[:45])
    tok = np.repeat(req_ad, req_len).astype(np.int32)
    widths = [(576, 832), (1088, 576), (832, 1088)][seed]
    b = workloads.Batch(f"random_{seed}", [torch.bfloat16, torch.float16, torch.bfloat16][seed], ranks, tok, req_ad,
                        req_len, int((req_len > 1).sum()), [("p", widths[0], widths[1]), ("q", widths[1], widths[0])],
                        seed=2000 + seed)
    _step_case(ops, b, [0, 1], layers=2)
