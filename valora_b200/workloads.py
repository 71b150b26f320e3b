"""Seeded synthetic workloads with the shapes and distributions of the five
benchmark configurations of the multi-LoRA batching operator.

Integers come from numpy.random.default_rng(seed) in the order
ranks -> text lengths -> adapter assignment; floats come from a torch
generator seeded with the same number, in the order (A, B per adapter per
projection) -> X -> Y0 (fp32, then cast).  Only shapes and distributions of
the serving traces are used; no trace or dataset item is reproduced.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import numpy as np
import torch

H = 4096
F = 11008
# (name, H_in, H_out) of the seven Qwen-VL-7B-shaped projections
PROJECTIONS: List[Tuple[str, int, int]] = [
    ("q", H, H), ("k", H, H), ("v", H, H), ("o", H, H),
    ("up", H, F), ("gate", H, F), ("down", F, H),
]
# which projection's activations each projection reads when a caller shares them:
# q, k, v read the layer input, up and gate the MLP input
SHARED_INPUT_OF: List[int] = [0, 0, 0, 3, 4, 4, 6]
ALPHA = 16.0


def zipf_probs(n: int, skew: float) -> np.ndarray:
    p = (np.arange(n, dtype=np.float64) + 1.0) ** (-skew)
    return p / p.sum()


@dataclass
class Batch:
    """One step's ragged batch: token -> adapter map in request order."""
    name: str
    dtype: torch.dtype
    ranks: np.ndarray                 # [n_adapters] true ranks
    tok_adapter: np.ndarray           # [T] int32 adapter id per token, batch order
    req_adapter: np.ndarray           # [n_req] adapter per request
    req_len: np.ndarray               # [n_req] tokens per request (1 for decode)
    n_prefill_req: int
    projections: List[Tuple[str, int, int]]
    layers: int = 1
    seed: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def T(self) -> int:
        return int(self.tok_adapter.shape[0])

    @property
    def n_adapters(self) -> int:
        return int(self.ranks.shape[0])

    def scalings(self) -> np.ndarray:
        return (ALPHA / self.ranks).astype(np.float32)

    def touched(self) -> np.ndarray:
        return np.unique(self.tok_adapter)

    def algorithmic_flops(self) -> int:
        """sum over problems and tokens of 2*r*(H_in+H_out): true ranks, true rows."""
        lr = int(self.ranks[self.tok_adapter].astype(np.int64).sum())
        per = sum(hi + ho for _, hi, ho in self.projections)
        return 2 * lr * per * self.layers

    def algorithmic_bytes(self, input_of=None) -> int:
        """X once, Y0 read + Y write, each touched adapter weight once (2-byte elements).
        input_of: projections that read another projection's X do not count it again."""
        e = 2
        act = sum((self.T * hi if input_of is None or input_of[p] == p else 0) + 2 * self.T * ho
                  for p, (_, hi, ho) in enumerate(self.projections)) * e
        rt = int(self.ranks[self.touched()].astype(np.int64).sum())
        wts = rt * sum(hi + ho for _, hi, ho in self.projections) * e
        return (act + wts) * self.layers


def _text_lengths(rng, n):
    v = np.rint(rng.lognormal(mean=4.5, sigma=0.8, size=n))
    return np.clip(v, 8, 1024).astype(np.int64)


def _tok_from_requests(req_adapter, req_len):
    return np.repeat(np.asarray(req_adapter, np.int32), np.asarray(req_len, np.int64)).astype(np.int32)


def config0() -> Batch:
    ranks = np.array([8, 16, 16, 32], np.int64)
    seg_len = np.array([37, 256, 1, 1, 120, 513], np.int64)
    seg_ad = np.array([0, 1, 2, 3, 1, 0], np.int32)
    return Batch("cfg0_ragged_fp16", torch.float16, ranks, _tok_from_requests(seg_ad, seg_len),
                 seg_ad, seg_len, len(seg_len), [("q", H, H)], seed=0)


def config1() -> Batch:
    rng = np.random.default_rng(1)
    ranks = np.full(64, 64, np.int64)
    req_ad = rng.choice(64, size=512, p=zipf_probs(64, 0.6)).astype(np.int32)
    return Batch("cfg1_decode_bgmv_bf16", torch.bfloat16, ranks, req_ad.copy(), req_ad,
                 np.ones(512, np.int64), 0, [("q", H, H)], seed=1)


def config2() -> Batch:
    rng = np.random.default_rng(2)
    ranks = rng.choice(np.array([8, 16, 32, 64, 128]), size=16).astype(np.int64)
    req_len = 256 + _text_lengths(rng, 24)
    req_ad = rng.choice(16, size=24, p=zipf_probs(16, 0.8)).astype(np.int32)
    return Batch("cfg2_prefill_hetero_fp16", torch.float16, ranks, _tok_from_requests(req_ad, req_len),
                 req_ad, req_len, 24, list(PROJECTIONS), seed=2)


def config3(layers: int = 32) -> Batch:
    rng = np.random.default_rng(3)
    ranks = np.full(64, 64, np.int64)
    pre_len = 256 + _text_lengths(rng, 8)
    n_dec = 384
    req_ad = rng.choice(64, size=8 + n_dec, p=zipf_probs(64, 0.8)).astype(np.int32)
    req_len = np.concatenate([pre_len, np.ones(n_dec, np.int64)])
    return Batch("cfg3_mixed_32x7_bf16", torch.bfloat16, ranks, _tok_from_requests(req_ad, req_len),
                 req_ad, req_len, 8, list(PROJECTIONS), layers=layers, seed=3)


def config4(n_gpus: int = 1, rank: int = 0, tokens: int = 16384, n_adapters: int = 1024) -> Batch:
    """Box-scale sweep.  The whole-box batch is generated once from seed 4; a
    GPU keeps the requests whose adapter it owns (adapter a lives on GPU
    a % n_gpus), in batch order."""
    rng = np.random.default_rng(4)
    ranks = rng.choice(np.array([16, 32, 64, 128]), size=n_adapters).astype(np.int64)
    n_pre_tok = tokens // 4
    # prefill segments: lengths as in config 2 until 25 % of the tokens are covered
    lens = []
    tot = 0
    while tot < n_pre_tok:
        L = int(256 + _text_lengths(rng, 1)[0])
        L = min(L, n_pre_tok - tot)
        lens.append(L)
        tot += L
    n_dec = tokens - tot
    req_len = np.concatenate([np.asarray(lens, np.int64), np.ones(n_dec, np.int64)])
    req_ad = rng.choice(n_adapters, size=req_len.shape[0], p=zipf_probs(n_adapters, 0.6)).astype(np.int32)
    n_pre = len(lens)
    if n_gpus > 1:
        keep = (req_ad % n_gpus) == rank
        n_pre = int(keep[:n_pre].sum())
        req_ad, req_len = req_ad[keep], req_len[keep]
    return Batch(f"cfg4_box_bf16_g{n_gpus}r{rank}", torch.bfloat16, ranks,
                 _tok_from_requests(req_ad, req_len), req_ad, req_len, n_pre, [("q", H, H)],
                 seed=4, extra={"n_gpus": n_gpus, "rank": rank})


CONFIGS = {0: config0, 1: config1, 2: config2, 3: config3, 4: config4}


def make_floats(batch: Batch, device="cpu", projections: Optional[List[int]] = None, layer: int = 0):
    """A/B per adapter per projection, then X and Y0 per projection (fp32 draws
    cast to the batch dtype).  Returns dict with
      A[p][a] [H_in, r], B[p][a] [r, H_out], X[p] [T, H_in], Y0[p] [T, H_out].
    On CPU the draw order is the one stated in the module docstring, seeded with
    batch.seed + 1000*layer; on a CUDA device each tensor is drawn by the device
    generator seeded the same way (bit patterns differ from the CPU draw)."""
    g = torch.Generator(device=device)
    g.manual_seed(batch.seed + 1000 * layer)
    sel = list(range(len(batch.projections))) if projections is None else projections
    A, B, X, Y0 = {}, {}, {}, {}

    def draw(shape, std):
        return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(batch.dtype)

    for p in sel:
        _, hi, ho = batch.projections[p]
        A[p], B[p] = [], []
        for a in range(batch.n_adapters):
            r = int(batch.ranks[a])
            A[p].append(draw((hi, r), 0.02))
            B[p].append(draw((r, ho), 0.02))
    for p in sel:
        _, hi, ho = batch.projections[p]
        X[p] = draw((batch.T, hi), 1.0)
    for p in sel:
        _, hi, ho = batch.projections[p]
        Y0[p] = draw((batch.T, ho), 1.0)
    return dict(A=A, B=B, X=X, Y0=Y0)
