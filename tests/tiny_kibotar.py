"""Tiny Kibotar configurations that differ in every size, constant and in the order of layers, and a writer of model
folders with seeded random weights (bfloat16 storage) whose scales make the attention sharp, the recurrent state's
memory long and the pair table, the step vectors, the shift and the gates matter, so that a wrong key, a window or a
block that is one token off, a lost state, a missing sink or a previous token that is forgotten shows.

A: latent attention (3 heads, key size 8, value size 12, latent 64), attention (4 query heads on 2 key heads, key 16,
   value 24, 8 of 16 numbers rotated with stretched frequencies, window 24, blocks of 4), gated linear attention (2 heads,
   key 16, value 24, rank 4); layers 1..2 run 3 times.
B: gated linear attention first and without a feed-forward; attention without a mask (every token seen, nothing pooled)
   and all numbers rotated, plain frequencies; attention with a window of 7 and blocks of 1; the whole model is the loop's
   span, twice.
C: sizes that are multiples of 4 but not of 8, an odd vocabulary; as many key heads as query heads; a window of one token
   with blocks of 2; one key head for 6 query heads without rotation, blocks (16) longer than the window (5); a window
   without blocks; a latent of 24 with one head; no loop at all; a table of pairs with one bucket.
D: sizes of the order of real models' heads (64), window 128 with blocks of 32, a loop of one pass.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import numpy as np
import torch


def _att(heads, kv_heads, dim, vdim, scale, rot=None, mask=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if len(rot) > 2:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), rot[2]))
    if mask is not None:
        m["mask"] = {"size": mask[0]}
        if mask[1] is not None:
            m["mask"]["pool"] = mask[1]
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _lat(heads, dim, vdim, kv_rank, scale, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}}


def _gla(heads, dim, vdim, tau, rank, mlp=None):
    # ("rank" is no key of a model folder's config: the loader takes it from a tensor's shape; the writer below reads it)
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _emb(scale, buckets, mul_prev, mul_cur):
    return {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}


CONFIGS: Dict[str, dict] = {
    "A": {"architecture": "Kibotar", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "embedding": _emb(0.7, 53, 31, 5),
          "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [_lat(3, 8, 12, 64, 0.6, _dense(96)),
                     _att(4, 2, 16, 24, 0.4, rot=(10000.0, 8, (8.0, 1.0, 4.0, 64)), mask=(24, 4), mlp=_dense(80)),
                     _gla(2, 16, 24, 8.0, 4, _dense(96))]},
    "B": {"architecture": "Kibotar", "vocab": 160, "width": 48, "norm": {"eps": 1e-6}, "embedding": _emb(1.0, 17, 3, 1),
          "loop": {"start": 0, "stop": 4, "times": 2},
          "layers": [_gla(3, 8, 16, 2.0, 8),
                     _att(2, 1, 24, 16, 0.3, rot=(500.0, 24), mlp=_dense(64)),
                     _att(3, 3, 8, 40, 0.5, rot=(77.0, 4, (2.0, 0.5, 2.0, 16)), mask=(7, 1), mlp=_dense(64)),
                     _lat(2, 16, 8, 64, 0.35)]},
    "C": {"architecture": "Kibotar", "vocab": 131, "width": 44, "norm": {"eps": 1e-5}, "embedding": _emb(0.25, 1, 9, 4),
          "layers": [_att(5, 5, 20, 12, 0.3, rot=(1000.0, 12), mask=(1, 2), mlp=_dense(52)),
                     _gla(1, 12, 20, 1.0, 3, _dense(36)),
                     _att(6, 1, 12, 28, 0.45, mask=(5, 16)),
                     _lat(1, 28, 12, 24, 0.25, _dense(60)),
                     _att(2, 2, 16, 16, 0.4, rot=(10000.0, 16), mask=(33, None), mlp=_dense(44)),
                     _gla(4, 4, 8, 32.0, 1)]},
    "D": {"architecture": "Kibotar", "vocab": 512, "width": 128, "norm": {"eps": 1e-5}, "embedding": _emb(0.6, 251, 64, 3),
          "loop": {"start": 2, "stop": 3, "times": 1},
          "layers": [_att(8, 4, 64, 32, 0.2, rot=(100000.0, 32, (8.0, 1.0, 2.0, 256)), mask=(128, 32), mlp=_dense(320)),
                     _gla(2, 64, 64, 12.0, 16, _dense(320)),
                     _lat(4, 64, 32, 128, 0.15, _dense(320))]},
}
SEEDS = {"A": 11, "B": 12, "C": 13, "D": 14}
PAGE = {"A": 16, "B": 8, "C": 16, "D": 32}


def random_tensors(cfg: dict, seed: int, overrides: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    t: Dict[str, torch.Tensor] = {}

    def mat(out, inp, gain=1.0):
        return torch.randn(out, inp, generator=g) * (gain / inp ** 0.5)

    def uni(n, lo, hi):
        return torch.rand(n, generator=g) * (hi - lo) + lo

    t["embed"] = torch.randn(V, W, generator=g)
    t["bigram"] = torch.randn(cfg["embedding"]["bigram"]["buckets"] + 1, W, generator=g) * 0.7
    if cfg.get("loop"):
        t["loop.step"] = torch.randn(cfg["loop"]["times"], W, generator=g) * 0.8
    t["final.norm"] = uni(W, 0.7, 1.3)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        t[p + "norm1"], t[p + "norm1b"] = uni(W, 0.7, 1.3), uni(W, 0.3, 0.7)
        t[p + "shift"] = uni(W, 0.1, 0.9)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            sharp = (4.0 / (m["scale"] * d ** 0.5)) ** 0.5            # scores of a few units: a sharp softmax
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * d, W, sharp), mat(G * d, W, sharp), mat(G * dv, W)
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                t[p + f"mix.{n}.b"] = torch.randn(rows, generator=g) * 0.3
            t[p + "mix.talk"] = torch.eye(H) * 0.7 + torch.randn(H, H, generator=g) * 0.3
            t[p + "mix.g"] = mat(H * dv, W, 2.0)
            t[p + "mix.o"], t[p + "mix.o.b"] = mat(W, H * dv, 0.8), torch.randn(W, generator=g) * 0.2
        elif L["type"] == "latent_attention":
            H, d, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            sharp = (4.0 / (m["scale"] * d ** 0.5)) ** 0.5
            t[p + "mix.q"], t[p + "mix.dkv"] = mat(H * d, W, sharp), mat(R, W)
            t[p + "mix.dkv.norm"] = uni(R, 0.7, 1.3)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * d, R, sharp), mat(H * dv, R)
            t[p + "mix.g"] = mat(H, W, 2.0)
            t[p + "mix.o"] = mat(W, H * dv, 0.8)
        else:
            H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["rank"]
            t[p + "mix.q"], t[p + "mix.k"] = mat(H * d, W, 1.5), mat(H * d, W, 1.5)
            t[p + "mix.v"], t[p + "mix.g"] = mat(H * dv, W, 1.5), mat(H * dv, W, 2.0)
            t[p + "mix.norm"] = uni(dv, 0.7, 1.3)
            t[p + "mix.a1"], t[p + "mix.a2"] = mat(r, W, 1.5), mat(H * d, r, 2.0)
            t[p + "mix.a2.b"] = uni(H * d, 0.0, 4.0)                   # decays from about a half (to the power 1/tau) to almost 1
            t[p + "mix.o"] = mat(W, H * dv, 0.8)
        if L["mlp"] is not None:
            t[p + "norm2"], t[p + "norm2b"] = uni(W, 0.7, 1.3), uni(W, 0.3, 0.7)
            t[p + "mlp.up"], t[p + "mlp.down"] = mat(L["mlp"]["ff"], W, 1.5), mat(W, L["mlp"]["ff"], 0.6)
    if overrides:
        for k, v in overrides.items():
            assert t[k].shape == v.shape, k
            t[k] = v
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def folder_config(cfg: dict) -> dict:
    """The config.json of a model folder: as ``cfg`` without the decay's rank, which a folder's tensors give."""
    out = json.loads(json.dumps(cfg))
    for L in out["layers"]:
        L["mixer"].pop("rank", None)
    return out


def write_model(cfg: dict, model_dir: str, seed: int, overrides: Optional[Dict[str, torch.Tensor]] = None) -> None:
    from safetensors.torch import save_file

    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(folder_config(cfg), f, indent=1)
    save_file(random_tensors(cfg, seed, overrides), os.path.join(model_dir, "model.safetensors"), metadata={"format": "pt"})


def read_model(model_dir: str):
    """(config dict, {name: float64 tensor}) for the plain implementation."""
    from safetensors.torch import load_file

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.double() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def prompts(cfg: dict, lengths: List[int], seed: int) -> List[List[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
