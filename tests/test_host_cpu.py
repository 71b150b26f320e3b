"""CPU-only checks: the C-ABI library loads and exports what the header
declares, host-side validation returns the documented codes, workload
generators and the schedule oracle are self-consistent."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from valora_b200 import _lib, workloads
from valora_b200.pool import AdapterPool


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _lib.declared_symbols()
    assert {"vlr_bgmv", "vlr_atmm", "vlr_pack", "vlr_lora_step", "vlr_var_len_copy"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n
    assert lib.vlr_version() >= 1


def test_host_validation_codes_without_a_gpu():
    lib = _lib.load()
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)
    # nothing is launched: validation fails first
    assert lib.vlr_bgmv(null, null, null, null, null, null, null, 0, null, 4, 4096, 64, 0, 0, null) == -1
    assert lib.vlr_bgmv(one, one, one, one, one, one, one, 0, one, 4, 4096, 64, 7, 0, null) == -3
    assert lib.vlr_bgmv(one, one, one, one, one, one, one, 0, one, 4, 4096, 256, 0, 0, null) == -2
    assert lib.vlr_bgmv(one, one, one, one, one, one, one, 0, one, 0, 4096, 64, 0, 0, null) == 0   # empty batch
    assert lib.vlr_atmm(one, one, one, one, one, one, one, 0, one, one, one, one, one, null, 0, 3,
                        100, 4096, 60, 10, 0, 0, null) == -2                                    # rank width % 8
    assert lib.vlr_atmm(one, one, one, one, one, one, one, 0, one, one, one, one, one, null, 0, 0,
                        100, 4096, 64, 10, 0, 0, null) == 0                                     # no problems
    assert lib.vlr_pack_workspace_bytes(1000, 64) > 0
    assert lib.vlr_pack(one, 10, one, 20000, 1, 128, 16, 8, one, one, one, one, one, one, 10, one, one,
                        one, 1 << 20, null) == -6                                               # too many adapters
    assert lib.vlr_pack(one, 10, one, 8, 1, 128, 16, 8, one, one, one, one, one, one, 10, one, one,
                        one, 16, null) == -5                                                    # workspace too small
    assert lib.vlr_step_plan_bytes(3) == 3 * lib.vlr_step_plan_bytes(1) > 0
    assert lib.vlr_lora_step(null, 2, 10, null, null, 0, 0, null, null, 4096, 4096, 64, 0, 15, null, 0, null,
                             null) == -1
    assert lib.vlr_pack(one, 10, one, 8, 1, 256, 16, 8, one, one, one, one, one, one, 10, one, one,
                        one, 1 << 20, null) == -6                                               # tile_m > 128
    assert lib.vlr_pack_static(one, 10, one, 8, 1, 128, 16, 64, one, one, one, one, one, one, 10, one, one,
                               null) == -6                                                      # 64 gathered rows per tile
    assert lib.vlr_pack_static(one, 9000, one, 8, 1, 128, 16, 8, one, one, one, one, one, one, 10, one, one,
                               null) == -9                                                      # beyond the built-in scratch
    assert lib.vlr_selftest_bounded_wait(0, null, null, null) == -6
    # fused base projection: y, x, w_base, v, v_pitch, wb_pool, cells_b, a_start_b, a_loc_b, slot_b, tiles,
    # counts, max_mma_tiles, T, h_in, h_out, dtype, dev_status, stream
    assert lib.vlr_fused_proj(one, one, null, one, 64, one, 8, one, one, 0, one, one, 0, 10, 4096, 4096, 1,
                              null, null) == -1                                                 # no base weight
    assert lib.vlr_fused_proj(one, one, one, one, 64, one, 8, one, one, 0, one, one, 0, 10, 4096, 4100, 1,
                              null, null) == -2                                                 # width % 64
    assert lib.vlr_fused_proj(one, one, one, one, 60, one, 8, one, one, 0, one, one, 0, 10, 4096, 4096, 1,
                              null, null) == -2                                                 # rank buffer pitch % 8
    assert lib.vlr_fused_proj(one, one, one, one, 64, one, 8, one, one, 0, one, one, 0, 0, 4096, 4096, 1,
                              null, null) == 0                                                  # empty batch
    assert b"workspace" in lib.vlr_error_string(-5)


def test_ops_refuse_cpu_tensors():
    from valora_b200 import ops
    x = torch.zeros(4, 64, dtype=torch.float16)
    z = torch.zeros(1, dtype=torch.int64)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.bgmv(torch.zeros(4, 16, dtype=torch.float16), x, torch.zeros(8, 1, 64, dtype=torch.float16),
                 z, z, z, torch.zeros(4, dtype=torch.int64), 0, torch.ones(1, dtype=torch.float16))


def test_workloads_are_deterministic_and_shaped():
    for i in range(5):
        a, b = workloads.CONFIGS[i](), workloads.CONFIGS[i]()
        assert np.array_equal(a.tok_adapter, b.tok_adapter) and np.array_equal(a.ranks, b.ranks)
    c0 = workloads.config0()
    assert c0.T == 928 and c0.algorithmic_flops() == 171_442_176 and c0.algorithmic_bytes() == 23_986_176
    c1 = workloads.config1()
    assert c1.T == 512 and c1.algorithmic_flops() == 536_870_912
    c3 = workloads.config3()
    assert c3.n_prefill_req == 8 and (c3.req_len[8:] == 1).all() and len(c3.req_len) == 392
    # shared activations: q/k/v and up/gate count their X once (three X tiles of 4096 columns fewer per layer)
    shared = c3.algorithmic_bytes(workloads.SHARED_INPUT_OF)
    assert c3.algorithmic_bytes() - shared == 3 * c3.T * 4096 * 2 * c3.layers
    assert c3.algorithmic_bytes(list(range(7))) == c3.algorithmic_bytes()
    c4 = workloads.config4()
    assert c4.T == 16384 and int((c4.req_len > 1).sum()) == c4.n_prefill_req
    # adapter-group sharding covers the whole box batch exactly once
    parts = [workloads.config4(n_gpus=4, rank=r) for r in range(4)]
    assert sum(p.T for p in parts) == c4.T
    for r, p in enumerate(parts):
        assert np.all(p.tok_adapter % 4 == r)


@pytest.mark.parametrize("cfg", [0, 1, 2, 3, 4])
def test_schedule_covers_every_token_once(cfg):
    b = workloads.CONFIGS[cfg]()
    pk = oracle.pack_sorted_ref(b.tok_adapter, b.ranks)
    tiles, grows, n_mma, n_g = oracle.tile_schedule_ref(b.tok_adapter, b.ranks, pk["perm"])
    seen = np.zeros(b.T, np.int32)
    for t in tiles:
        kind, a, r, first, n = t[:5]
        rows = np.arange(first, first + n) if kind == 0 else grows[first:first + n]
        assert np.all(b.tok_adapter[rows] == a) and r == b.ranks[a]
        seen[rows] += 1
    assert np.all(seen == 1)
    assert int(pk["seg_len"].sum()) == b.T and np.all(np.diff(pk["seg_adapter"]) > 0)


def test_pool_allocator_matches_reference_semantics():
    pool = AdapterPool(cells=64, width=8, n_slots=4, dtype=torch.float16, device="cpu")
    state = np.ones(64, np.uint8)
    a = pool.alloc(10); ra = oracle.alloc_ref(state, 10)
    b = pool.alloc(7); rb = oracle.alloc_ref(state, 7)
    pool.free(a[2:6]); state[ra[2:6]] = 1
    c = pool.alloc(9); rc = oracle.alloc_ref(state, 9)
    assert np.array_equal(a, ra) and np.array_equal(b, rb) and np.array_equal(c, rc)
    assert np.array_equal(pool.mem_state, state)
    run = pool.alloc_contiguous(12)
    assert np.array_equal(run, np.arange(run[0], run[0] + 12)) and np.all(state[run] == 1)
    with pytest.raises(Exception):
        pool.alloc(1000)


def test_launcher_follows_the_tile_table():
    """The launch-level choices come from the committed table (valora_b200/tile_table.json,
    written by the autotuner): for every entry the launcher reports exactly the entry's
    values, rank bounds in between resolve to the next entry up, a replaced table is
    honoured at once and a table the kernels cannot run is refused."""
    import json
    from valora_b200 import tile_table
    lib = _lib.load()
    t = tile_table.load(tile_table.DEFAULT_PATH)
    assert t["gpu"] and len(t["entries"]) >= 4
    tile_table.apply(lib, t)
    for e in t["entries"]:
        got = tile_table.choice(lib, bool(e["step"]), e["max_rank"])
        keys = ("shrink_stages", "expand_stages", "small_call_rows", "wide_gather_below_rank")
        assert {k: got[k] for k in keys} == {k: e[k] for k in keys}, e
    by = {(e["step"], e["max_rank"]): e for e in t["entries"]}
    assert tile_table.choice(lib, True, 16)["shrink_stages"] == by[(1, 64)]["shrink_stages"]
    assert tile_table.choice(lib, True, 96)["shrink_stages"] == by[(1, 128)]["shrink_stages"]
    assert tile_table.choice(lib, False, 8)["small_call_rows"] == by[(0, 64)]["small_call_rows"]
    other = json.loads(json.dumps(t))
    other["entries"][0].update(shrink_stages=2, small_call_rows=64)
    tile_table.apply(lib, other)
    e0 = other["entries"][0]
    assert tile_table.choice(lib, bool(e0["step"]), e0["max_rank"])["shrink_stages"] == 2
    bad = json.loads(json.dumps(t))
    bad["entries"][1].update(expand_stages=4)            # rank 128 does not fit 48 KB expand stages
    with pytest.raises(RuntimeError):
        tile_table.apply(lib, bad)
    tile_table.apply(lib, t)
    assert tile_table.choice(lib, bool(e0["step"]), e0["max_rank"])["shrink_stages"] == t["entries"][0]["shrink_stages"]
    eng = t["engine"]
    assert eng["gather_rows_per_tile"] <= 32 and eng["mma_min_rows"] >= 1


def test_python_constants_mirror_the_header():
    """The flag and layout values the Python layer passes are the header's `#define`s."""
    import os
    import re
    from valora_b200 import ops
    hdr = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "vlr.h")).read()
    defs = {m.group(1): int(m.group(2), 0) for m in re.finditer(r"#define\s+(VLR_\w+)\s+(-?\d+)\b", hdr)}
    pairs = {
        "VLR_F16": ops.F16, "VLR_BF16": ops.BF16, "VLR_LAYOUT_PUNICA": ops.LAYOUT_PUNICA, "VLR_LAYOUT_ROWS": ops.LAYOUT_ROWS,
        "VLR_ATMM_ACCUMULATE_SHRINK": ops.ATMM_ACCUMULATE_SHRINK, "VLR_ATMM_APPLY_SCALE": ops.ATMM_APPLY_SCALE,
        "VLR_ATMM_FULL_TILES": ops.ATMM_FULL_TILES, "VLR_TILE_INTS": ops.TILE_INTS, "VLR_COUNT_INTS": ops.COUNT_INTS,
        "VLR_PHASE_SHRINK_MMA": ops.PHASE_SHRINK_MMA, "VLR_PHASE_SHRINK_GATHER": ops.PHASE_SHRINK_GATHER,
        "VLR_PHASE_EXPAND_MMA": ops.PHASE_EXPAND_MMA, "VLR_PHASE_EXPAND_GATHER": ops.PHASE_EXPAND_GATHER,
        "VLR_STEP_GATHER_ON_TENSOR_CORES": ops.STEP_GATHER_ON_TENSOR_CORES,
        "VLR_STEP_WIDE_GATHER_STAGES": ops.STEP_WIDE_GATHER_STAGES,
        "VLR_STEP_ALL_WIDE_GATHER_STAGES": ops.STEP_ALL_WIDE_GATHER_STAGES,
        "VLR_STEP_SPLIT_RANK_CLASSES": ops.STEP_SPLIT_RANK_CLASSES,
    }
    for name, val in pairs.items():
        assert name in defs, name
        assert defs[name] == val, name
    # the step's flags are distinct bits above the four phase bits
    bits = [ops.STEP_GATHER_ON_TENSOR_CORES, ops.STEP_WIDE_GATHER_STAGES, ops.STEP_ALL_WIDE_GATHER_STAGES,
            ops.STEP_SPLIT_RANK_CLASSES]
    assert len(set(bits)) == 4 and all(b & ops.PHASE_ALL == 0 and b & (b - 1) == 0 for b in bits)
