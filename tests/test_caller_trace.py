"""The reference's own caller code drives the drop-in entry points.

tests/golden/caller_trace.{json,npz} is the list of operator calls that the
methods _lora_get_qkv, _lora_get_o, _batch_lora_get_qkv and _batch_lora_get_o of
the reference's LoraUnorderedBatchInfer made when their unmodified source was
executed on CPU (tests/golden/make_caller_trace.py): which tensor and which view
of it went into which argument, the slot numbers, the tile integers.  Here that
list is replayed - through the oracle on CPU (must reproduce the recorded
outputs bit for bit) and through the installed module names `atmm_ops` and
`valora._kernels` on a GPU (every call within tolerance of the oracle on the
same inputs, and the methods' results q / k / v / o within tolerance of the
recorded ones)."""
import json
import os

import numpy as np
import pytest
import torch

from tests.helpers import oracle_dispatch_bgmv, oracle_dispatch_sgmm, out_tolerance

HERE = os.path.dirname(os.path.abspath(__file__))
DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "int64": torch.int64, "int8": torch.int8}


def _load():
    doc = json.load(open(os.path.join(HERE, "golden", "caller_trace.json")))
    arr = np.load(os.path.join(HERE, "golden", "caller_trace.npz"))
    return doc, arr


def _tensor(a, dtype, device):
    if dtype in (torch.float16, torch.bfloat16):
        return torch.from_numpy(a.view(np.int16).copy()).view(dtype).to(device)
    return torch.from_numpy(a.copy()).to(device)


def _state(scene, arr, tag, device):
    return {n: _tensor(arr[f"{tag}/init/{n}"], DT[m["dtype"]], device) for n, m in scene["tensors"].items()}


def _args(call, state):
    out = []
    for a in call["args"]:
        if "t" in a:
            out.append(torch.as_strided(state[a["t"]], a["shape"], a["stride"], a["off"]))
        elif "none" in a:
            out.append(None)
        else:
            out.append(a["i"])
    return out


def _replay(scene, arr, tag, device, impls, per_call=None):
    state = _state(scene, arr, tag, device)
    for call in scene["calls"]:
        if call["fn"] == "host_write":
            state[call["t"]].copy_(_tensor(arr[f"{tag}/{call['array']}"], state[call["t"]].dtype, device))
            continue
        args = _args(call, state)
        if per_call is not None:
            before = [a.detach().cpu().clone() if isinstance(a, torch.Tensor) else a for a in args]
        impls[call["fn"]](*args)
        if per_call is not None:
            per_call(call, before, args[0])
    return state


def test_trace_has_the_callers_binding():
    """What the reference's methods do with the two entry points, read off the recorded list."""
    doc, _ = _load()
    pre, dec = doc["scenes"]["prefill"], doc["scenes"]["decode"]
    calls = [c for c in pre["calls"] if c["fn"] != "host_write"]
    assert [c["fn"] for c in calls] == ["dispatch_sgmm"] * 8
    assert [c["args"][7]["i"] for c in calls] == [0, 1, 2, 0, 1, 2, 3, 3]         # three shrinks, three expands, then o
    assert [c["args"][0]["t"] for c in calls[:3]] == ["delta0", "delta1", "delta2"]
    assert calls[4]["args"][0]["t"] == "cache_k" and calls[5]["args"][0]["t"] == "cache_v"
    assert calls[6]["args"][0]["t"] == "delta0" and calls[6]["args"][1]["t"] == "attn_out"   # o reuses delta[0]
    for c in calls:
        tiles = [a["i"] for a in c["args"][15:21]]
        assert tiles[5] == tiles[2]                        # tb_z is passed where the sixth tile integer belongs
    dcalls = [c for c in dec["calls"] if c["fn"] != "host_write"]
    # decode: q and k go through BGMV, v through ATMM - on the same value_buffer - and o through BGMV
    assert [c["fn"] for c in dcalls] == ["dispatch_bgmv"] * 4 + ["dispatch_sgmm"] * 2 + ["dispatch_bgmv"] * 2
    assert {c["args"][2]["t"] for c in dcalls if c["args"][1]["t"].startswith("delta")} == {"value_buffer"}
    assert dcalls[0]["args"][6]["t"] == "req_bins" and calls[0]["args"][6]["t"] == "batch_req_bins"


def test_oracle_replay_reproduces_the_recorded_results():
    doc, arr = _load()
    impls = {"dispatch_sgmm": oracle_dispatch_sgmm, "dispatch_bgmv": oracle_dispatch_bgmv}
    for tag, scene in doc["scenes"].items():
        state = _replay(scene, arr, tag, "cpu", impls)
        for n in scene["written"]:
            want = _tensor(arr[f"{tag}/final/{n}"], state[n].dtype, "cpu")
            assert torch.equal(state[n].view(torch.int16), want.view(torch.int16)), (tag, n)


@pytest.mark.gpu
def test_gpu_replay_through_the_installed_modules():
    from valora_b200 import dropin, ops
    dropin.install(force=True)
    from atmm_ops import dispatch_bgmv as dispatch_sgmm
    from valora._kernels import dispatch_bgmv
    doc, arr = _load()
    cpu_impl = {"dispatch_sgmm": oracle_dispatch_sgmm, "dispatch_bgmv": oracle_dispatch_bgmv}
    worst = [0.0]

    def per_call(call, before, out):
        # the oracle on exactly what the GPU call was given, fp32 result
        ref = cpu_impl[call["fn"]](*before, rounding="fp32")
        err = (out.float().cpu() - ref).abs() - out_tolerance(ref, out.dtype)
        worst[0] = max(worst[0], float(err.max()))
        assert float(err.max()) <= 0.0, (call["fn"], call["args"][0]["t"], call["args"][7]["i"])

    for tag, scene in doc["scenes"].items():
        state = _replay(scene, arr, tag, "cuda:0", {"dispatch_sgmm": dispatch_sgmm, "dispatch_bgmv": dispatch_bgmv},
                        per_call=per_call)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        for n in scene["written"]:
            want = _tensor(arr[f"{tag}/final/{n}"], state[n].dtype, "cpu").float()
            got = state[n].float().cpu()
            # the recorded results are 16-bit values that went through the same two roundings
            assert float(((got - want).abs() - 2 * out_tolerance(want, state[n].dtype)).max()) <= 0.0, (tag, n)
        # what the methods returned
        for name in ("q", "o"):
            assert scene["returned"][name]["t"] in scene["written"]
