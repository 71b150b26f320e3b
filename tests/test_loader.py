"""HF PEFT adapter directory -> pool blocks (CPU) and -> a running engine (GPU)."""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from valora_b200 import loader, workloads

MODULES = ["q_proj", "v_proj", "up_proj"]
WIDTHS = [(64, 64), (64, 64), (64, 192)]                  # (in, out) per module


def _write_adapter(path, r, alpha, layers, fmt, seed, skip=()):
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"r": r, "lora_alpha": alpha, "target_modules": MODULES, "peft_type": "LORA"}, f)
    g = torch.Generator().manual_seed(seed)
    w = {}
    for l in range(layers):
        for m, (hi, ho) in zip(MODULES, WIDTHS):
            if (l, m) in skip:
                continue
            sub = "self_attn" if m.endswith("_proj") and m[0] in "qkvo" else "mlp"
            base = f"base_model.model.model.layers.{l}.{sub}.{m}"
            w[f"{base}.lora_A.weight"] = torch.randn(r, hi, generator=g) * 0.1
            w[f"{base}.lora_B.weight"] = torch.randn(ho, r, generator=g) * 0.1
    # a key of layer 1 must not be mistaken for layer 11 and vice versa
    w["base_model.model.model.layers.11.self_attn.q_proj.lora_A.weight"] = torch.zeros(r, 64)
    w["base_model.model.model.layers.11.self_attn.q_proj.lora_B.weight"] = torch.zeros(64, r)
    if fmt == "safetensors":
        from safetensors.torch import save_file
        save_file(w, os.path.join(path, "adapter_model.safetensors"))
    else:
        torch.save(w, os.path.join(path, "adapter_model.bin"))
        torch.save({"lr": 1e-4}, os.path.join(path, "training_args.bin"))      # must be ignored
    return w


@pytest.mark.parametrize("fmt", ["bin", "safetensors"])
def test_read_and_blocks(tmp_path, fmt):
    w = _write_adapter(str(tmp_path / "ad"), 16, 32, 2, fmt, seed=1, skip={(1, "up_proj")})
    cfg, got = loader.read_adapter(str(tmp_path / "ad"))
    assert loader.lora_rank(cfg) == 16 and loader.lora_scaling(cfg) == 2.0
    assert set(got) == set(w) and all(torch.equal(got[k], w[k]) for k in w)
    wi, wo = [a for a, _ in WIDTHS], [b for _, b in WIDTHS]
    for layout in ("rows", "punica"):
        a_blocks, b_blocks = loader.pool_blocks(got, cfg, 1, MODULES, wi, wo, torch.float16, b_layout=layout)
        assert a_blocks[2] is None and b_blocks[2] is None                      # module the adapter skips
        A = w["base_model.model.model.layers.1.self_attn.q_proj.lora_A.weight"]
        B = w["base_model.model.model.layers.1.self_attn.q_proj.lora_B.weight"]
        assert torch.equal(a_blocks[0], A.half())                               # cell j = row j of A^T
        if layout == "rows":
            assert torch.equal(b_blocks[0], B.half().t().contiguous())          # cell k = row k of B
        else:
            # flat bytes of [out, r]; the oracle's packer states the same layout
            want = oracle.pack_w_combined_ref([A.t().contiguous().half(), None, None, None],
                                              [B.t().contiguous().half(), None, None, None], 16, 4)
            assert torch.equal(b_blocks[0].reshape(-1), B.half().reshape(-1))
            assert torch.equal(want[1][:16].reshape(16, 64), b_blocks[0])
            assert torch.equal(want[0][:16].reshape(16, 64), a_blocks[0])
    with pytest.raises(ValueError):
        loader.pool_blocks(got, cfg, 0, MODULES, [64, 64, 32], wo, torch.float16)   # wrong width
    with pytest.raises(FileNotFoundError):
        loader.read_adapter(str(tmp_path / "nothing"))


@pytest.mark.gpu
def test_engine_runs_a_loaded_adapter(tmp_path):
    from valora_b200 import ops
    from valora_b200.engine import LoraStepEngine
    dev = "cuda:0"
    layers, ranks = 2, np.array([8, 16, 16])
    projs = [(m, hi, ho) for m, (hi, ho) in zip(MODULES, WIDTHS)]
    eng = LoraStepEngine(projs, ranks, (workloads.ALPHA / ranks).astype(np.float32), torch.float16, dev, layers, 300)
    eng.randomize_weights(seed=3)
    w = _write_adapter(str(tmp_path / "ad"), 16, 8, layers, "safetensors", seed=5)
    side = torch.cuda.Stream()
    done = loader.load_into_engine(eng, 1, str(tmp_path / "ad"), MODULES, stream=side)
    torch.cuda.current_stream().wait_event(done)
    with pytest.raises(ValueError):
        loader.load_into_engine(eng, 0, str(tmp_path / "ad"), MODULES)           # slot 0 has rank 8
    tok = np.concatenate([np.full(200, 1), np.full(37, 2), [1, 1, 0, 2, 1]]).astype(np.int64)
    T = tok.shape[0]
    g = torch.Generator().manual_seed(2)
    X = [[torch.randn(T, hi, generator=g).half() for _, hi, _ in projs] for _ in range(layers)]
    Y0 = [[torch.randn(T, ho, generator=g).half() for _, _, ho in projs] for _ in range(layers)]
    for l in range(layers):
        for p in range(len(projs)):
            eng.x[l][p][:T].copy_(X[l][p])
            eng.y[l][p][:T].copy_(Y0[l][p])
    eng.step(torch.from_numpy(tok).to(dev))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    rows = torch.from_numpy(np.nonzero(tok == 1)[0])
    for l in range(layers):
        for p, m in enumerate(MODULES):
            sub = "self_attn" if m[0] in "qkvo" else "mlp"
            A = w[f"base_model.model.model.layers.{l}.{sub}.{m}.lora_A.weight"].half()      # [r, in]
            B = w[f"base_model.model.model.layers.{l}.{sub}.{m}.lora_B.weight"].half()      # [out, r]
            v = (X[l][p][rows].float() @ A.float().t()).half().float()
            want = Y0[l][p][rows].float() + (v @ B.float().t()) * 0.5                       # alpha / r = 8 / 16
            got = eng.y[l][p][:T].float().cpu()[rows]
            assert float((got - want).abs().max()) <= 2e-2, (l, m)
