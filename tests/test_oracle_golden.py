"""The oracle against the golden vectors produced by running the reference's
own Python (tests/golden/make_golden.py).  CPU only."""
import hashlib
import os

import numpy as np
import pytest
import torch

import oracle
from oracle.pack_ref import FILL_N
from valora_b200 import workloads

G = os.path.join(os.path.dirname(__file__), "golden")


def _t(a, dtype):
    return torch.from_numpy(a.view(np.int16).copy()).view(dtype)


def _u16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("tag,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_groupgemm_small_bit_exact(tag, dtype):
    z = np.load(os.path.join(G, "groupgemm.npz"))
    x, y0 = _t(z[f"{tag}_x"], dtype), _t(z[f"{tag}_y0"], dtype)
    wa, wb = _t(z[f"{tag}_wa"], dtype), _t(z[f"{tag}_wb"], dtype)
    seg_len, seg_ad = z["seg_len"], z["seg_ad"]
    v = torch.zeros(x.shape[0], wa.shape[1], dtype=dtype)
    oracle.groupgemm_ref(v, x, wa, seg_ad, seg_len, 1.0, "shrink")
    assert np.array_equal(_u16(v), z[f"{tag}_v"])
    y = y0.clone()
    oracle.groupgemm_ref(y, v, wb, seg_ad, seg_len, float(z["expand_scaling"][0]), "expand")
    assert np.array_equal(_u16(y), z[f"{tag}_y"])


@pytest.mark.parametrize("tag,dtype", [("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_segment_walk_matches_groupgemm_golden(tag, dtype):
    """The per-segment mm(mm(x, A), B) * s walk and the fp32 truth agree with the
    reference-produced output within the 16-bit rounding of the intermediate."""
    z = np.load(os.path.join(G, "groupgemm.npz"))
    x, y0 = _t(z[f"{tag}_x"], dtype), _t(z[f"{tag}_y0"], dtype)
    wa, wb = _t(z[f"{tag}_wa"], dtype), _t(z[f"{tag}_wb"], dtype)
    ranks = z["ranks"]
    A = [wa[a, :r].T.contiguous() for a, r in enumerate(ranks)]
    B = [wb[a, :, :r].T.contiguous() for a, r in enumerate(ranks)]
    s = float(z["expand_scaling"][0])
    y32 = oracle.ragged_lora_ref_fp32(y0, x, A, B, z["seg_len"], z["seg_ad"], [s] * 4)
    gold = _t(z[f"{tag}_y"], dtype)
    tol = 2e-3 if dtype == torch.float16 else 1.6e-2   # one ulp of the output near |y| ~ 4
    assert float((y32 - gold.float()).abs().max()) <= tol
    y16 = oracle.ragged_lora_ref(y0, x, A, B, z["seg_len"], z["seg_ad"], [s] * 4)
    assert float((y16.float() - gold.float()).abs().max()) <= 2 * tol


def test_config0_digest():
    """Full config 0 through the oracle reproduces the reference's bytes."""
    torch.set_num_threads(1)
    z = np.load(os.path.join(G, "groupgemm.npz"))
    b = workloads.config0()
    fl = workloads.make_floats(b)
    R = int(b.ranks.max())
    wa = torch.zeros(b.n_adapters, R, 4096, dtype=b.dtype)
    wb = torch.zeros(b.n_adapters, 4096, R, dtype=b.dtype)
    for a in range(b.n_adapters):
        r = int(b.ranks[a])
        wa[a, :r] = fl["A"][0][a].T
        wb[a, :, :r] = fl["B"][0][a].T
    v = torch.zeros(b.T, R, dtype=b.dtype)
    oracle.groupgemm_ref(v, fl["X"][0], wa, b.req_adapter, b.req_len, 1.0, "shrink")
    assert hashlib.sha256(_u16(v).tobytes()).digest() == z["cfg0_v_sha256"].tobytes()
    y = fl["Y0"][0].clone()
    start = 0
    for L, a in zip(b.req_len.tolist(), b.req_adapter.tolist()):
        oracle.groupgemm_ref(y[start:start + L], v[start:start + L], wb, [a], [L],
                             float(workloads.ALPHA / b.ranks[a]), "expand")
        start += L
    assert np.array_equal(_u16(y[:4, :64]), z["cfg0_y_head"])
    assert hashlib.sha256(_u16(y).tobytes()).digest() == z["cfg0_y_sha256"].tobytes()
    # and the fp32 truth of the operator contract sits within tolerance of it
    y32 = oracle.ragged_lora_ref_fp32(fl["Y0"][0], fl["X"][0], fl["A"][0], fl["B"][0],
                                      b.req_len, b.req_adapter, b.scalings())
    assert float((y32 - y.float()).abs().max()) <= 1e-2


def _pack_cases():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(G, "make_golden.py"))
    src = open(os.path.join(G, "make_golden.py")).read()
    # only the PACK_CASES literal is needed; avoid executing the generator
    start = src.index("PACK_CASES = [")
    end = src.index("]\n\n\ndef gen_pack")
    ns = {}
    exec(src[start:end + 1], ns)
    return ns["PACK_CASES"]


def test_set_sgmm_args_bit_exact():
    z = np.load(os.path.join(G, "set_sgmm_args.npz"))
    for ci, (dirs, lens, merged) in enumerate(_pack_cases()):
        for is_prefill in (True, False):
            tag = f"c{ci}_{'p' if is_prefill else 'd'}"
            oc, li, si, npb = oracle.set_sgmm_args_ref(dirs, lens, is_prefill, merged)
            assert np.array_equal(oc, z[tag + "_output_counts"]), tag
            assert np.array_equal(li, z[tag + "_lora_ids"]), tag
            assert np.array_equal(si, z[tag + "_start_ids"]), tag
            assert [npb[0], npb[1][0], npb[1][1]] == z[tag + "_num_problems"].tolist(), tag


def test_rle_agrees_with_host_packer():
    """Token-level run-length encoding (the intended device packer) gives the host
    packer's counts and offsets when the same batch is described per token."""
    z = np.load(os.path.join(G, "set_sgmm_args.npz"))
    for ci, (dirs, lens, merged) in enumerate(_pack_cases()):
        if merged is not None:
            continue
        names = sorted(set(dirs))
        ids = np.asarray([names.index(d) for d in dirs])
        a_len = np.full(len(names), 64 * 4)
        for is_prefill in (True, False):
            tag = f"c{ci}_{'p' if is_prefill else 'd'}"
            tok = np.repeat(ids, lens) if is_prefill else ids
            r = oracle.rle_ref(tok, a_len)
            P = int(z[tag + "_num_problems"][0])
            assert r["P"] == P
            assert np.array_equal(r["seg_len"], z[tag + "_output_counts"][:P])
            if len(dirs) > 1:
                assert np.array_equal(r["seg_start"], z[tag + "_start_ids"][:P + 1])
            else:
                assert r["seg_start"][0] == z[tag + "_start_ids"][0] == 0
            assert np.all(r["seg_rank"] == 64)
            assert np.array_equal(r["seg_adapter"], ids[np.concatenate([[True], ids[1:] != ids[:-1]])])


def test_mem_allocator_bit_exact():
    z = np.load(os.path.join(G, "mem_allocator.npz"))
    state = np.ones(64, np.uint8)
    a = oracle.alloc_ref(state, 10)
    b = oracle.alloc_ref(state, 7)
    state[a[2:6]] = 1
    c = oracle.alloc_ref(state, 9)
    state[b] = 1
    d = oracle.alloc_ref(state, 12)
    for name, val in dict(a=a, b=b, c=c, d=d).items():
        assert np.array_equal(val, z[name]), name
    assert np.array_equal(state, z["state"])
    assert int(state.sum()) == int(z["can_use"][0])
    with pytest.raises(Exception):
        oracle.alloc_ref(state, 1000)
    assert int(z["raised"][0]) == 1
