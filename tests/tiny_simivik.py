"""Tiny Simivik configurations that differ in every size, constant and in the order of layers, and a writer of model
folders with seeded random weights (bfloat16 storage) whose scales make the attention sharp and the scores reach the
cap, the lightning state's memory long, and the routers' choices clear, so that a wrong key, a window that is one
token off, a lost state, a missing first token or a wrong expert shows.

A: attention first (4 query heads on 2 key heads, key size 16, value size 24, 3 taps, 8 of 16 numbers rotated, window 24
   keeping 5, cap 5) with a dense feed-forward; lightning (key size 16, value size 24) with 6 experts of which 2 are
   used and a shared one; then each once more on the same tensors with a cache of its own.
B: lightning first, without a feed-forward; attention without convolution, cap or window, all numbers rotated;
   a window of 7 that keeps nothing behind 2 taps; experts without a shared one (3 of 5); a window wider than any prompt.
C: sizes that are multiples of 4 but not of 8, an odd vocabulary; as many key heads as query heads; one tap; a window of
   one token that keeps one; one lightning head with decay 1; all 3 of 3 experts; one key head for 6 query heads, no
   rotation, 8 taps, more kept tokens (40) than the window (33), a cap of 1.5.
D: sizes of the order of real models' heads (64), 8 experts of which 2, a window of 128 keeping 16.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import numpy as np
import torch


def _att(heads, kv_heads, dim, vdim, scale, conv=None, rot=None, mask=None, softcap=None, mlp=None, weights_of=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if softcap is not None:
        m["softcap"] = softcap
    e = {"type": "attention", "mixer": m, "mlp": mlp}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def _lin(heads, dim, vdim, decay, mlp=None, weights_of=None):
    e = {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


_A0 = dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, conv=3, rot=(10000.0, 8), mask=(24, 5), softcap=5.0, mlp=_dense(96))
_A1 = dict(heads=2, dim=16, vdim=24, decay=(0.9, 0.995), mlp=_moe(6, 2, 32, 48))

CONFIGS: Dict[str, dict] = {
    "A": {"architecture": "Simivik", "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
          "layers": [_att(**_A0), _lin(**_A1), _att(**_A0, weights_of=0), _lin(**_A1, weights_of=1)]},
    "B": {"architecture": "Simivik", "vocab": 300, "width": 96, "norm": {"eps": 1e-6},
          "layers": [_lin(3, 8, 40, (0.5, 0.97, 0.9999)),
                     _att(2, 1, 24, 16, 0.2, rot=(500.0, 24), mlp=_dense(72)),
                     _att(3, 3, 8, 40, 0.35, conv=2, rot=(77.0, 4), mask=(7, 0), softcap=30.0, mlp=_moe(5, 3, 40)),
                     _att(6, 2, 8, 8, 0.35, conv=4, rot=(10000.0, 8), mask=(1000, 3), mlp=_dense(130))]},
    "C": {"architecture": "Simivik", "vocab": 257, "width": 100, "norm": {"eps": 3e-5},
          "layers": [_att(5, 5, 20, 12, 0.22, conv=1, rot=(1000.0, 12), mask=(1, 1), softcap=8.0, mlp=_dense(76)),
                     _lin(1, 12, 20, (1.0,), mlp=_moe(3, 3, 28, 36)),
                     _att(6, 1, 12, 28, 0.3, conv=8, mask=(33, 40), softcap=1.5),
                     _lin(5, 4, 4, (0.3, 0.8, 0.95, 0.99, 0.999), mlp=_dense(52))]},
    "D": {"architecture": "Simivik", "vocab": 512, "width": 256, "norm": {"eps": 1e-5},
          "layers": [_att(8, 2, 64, 64, 0.125, conv=4, rot=(100000.0, 32), mask=(128, 16), softcap=30.0, mlp=_moe(8, 2, 128, 256)),
                     _lin(4, 64, 32, (0.8, 0.95, 0.99, 0.999), mlp=_dense(512)),
                     _att(4, 4, 32, 128, 0.18, conv=3, rot=(10000.0, 32), mask=(64, 4), mlp=_dense(384))]},
}
SEEDS = {"A": 3, "B": 5, "C": 8, "D": 13}
PAGE = {"A": 16, "B": 8, "C": 16, "D": 32}


def _owner(cfg: dict, i: int) -> int:
    while "weights_of" in cfg["layers"][i]:
        i = cfg["layers"][i]["weights_of"]
    return i


def _route_dims(cfg: dict) -> int:
    """The residual stream's last numbers carry, per token of the vocabulary, one clear level per expert."""
    return max([L["mlp"]["router"]["experts"] for L in cfg["layers"] if L["mlp"] and L["mlp"]["kind"] == "moe"] or [0])


def random_tensors(cfg: dict, seed: int, overrides: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    R = _route_dims(cfg)
    t: Dict[str, torch.Tensor] = {}

    def mat(out, inp, gain=1.0):
        return torch.randn(out, inp, generator=g) * (gain / inp ** 0.5)

    def uni(n, lo, hi):
        return torch.rand(n, generator=g) * (hi - lo) + lo

    def quiet(m):
        """A matrix that writes into the residual stream leaves the routing numbers almost alone."""
        if R:
            m[W - R:] *= 0.05
        return m

    emb = torch.randn(V, W, generator=g)
    if R:       # every token ranks the experts in an order of its own, a level apart
        levels = torch.arange(R, dtype=torch.float32) - (R - 1) / 2
        for v in range(V):
            emb[v, W - R:] = levels[torch.randperm(R, generator=g)] * 1.2
    t["embed"] = emb
    t["final.norm"] = uni(W, -0.2, 0.2)
    for i, L in enumerate(cfg["layers"]):
        if "weights_of" in L:
            continue
        p, m = f"l{i}.", L["mixer"]
        t[p + "norm1"] = uni(W, -0.2, 0.2)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            sharp = (4.0 / (m["scale"] * d ** 0.5)) ** 0.5            # scores of a few units: a sharp softmax, up to the cap
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * d, W, sharp), mat(G * d, W, sharp), mat(G * dv, W)
            if m.get("conv"):
                for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                    w = torch.randn(rows, m["conv"], generator=g) * (0.5 / m["conv"] ** 0.5)
                    w[:, -1] += 0.8                                     # mostly the row itself
                    t[p + f"mix.{n}.conv"] = w
            t[p + "mix.o"] = quiet(mat(W, H * dv, 0.8))
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = mat(H * d, W, 1.5), mat(H * d, W, 1.5)
            t[p + "mix.v"], t[p + "mix.g"] = mat(H * dv, W, 1.5), mat(H * dv, W, 2.0)
            t[p + "mix.norm"] = uni(H * dv, 0.7, 1.3)
            t[p + "mix.o"] = quiet(mat(W, H * dv, 0.8))
        mlp = L["mlp"]
        if mlp is None:
            continue
        t[p + "norm2"] = uni(W, -0.2, 0.2)
        if mlp["kind"] == "dense":
            t[p + "mlp.up"], t[p + "mlp.down"] = mat(mlp["ff"], W, 1.5), quiet(mat(W, mlp["ff"], 0.6))
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            t[p + "norm2"][W - R:] = 0.0                                # (the levels reach the router as they are)
            router = mat(E, W, 0.1)
            router[:, W - R:] = 0.0
            router[:, W - R:W - R + E] += torch.eye(E) * min(5.0, 16.0 / R)          # reads the token's level for this expert
            t[p + "mlp.router"] = router
            for e in range(E):
                t[p + f"mlp.e{e}.gate"], t[p + f"mlp.e{e}.up"] = mat(ff, W, 1.5), mat(ff, W, 1.5)
                t[p + f"mlp.e{e}.down"] = quiet(mat(W, ff, 1.0))
            if mlp.get("shared"):
                S = mlp["shared"]["ff"]
                t[p + "mlp.shared.gate"], t[p + "mlp.shared.up"] = mat(S, W, 1.5), mat(S, W)
                t[p + "mlp.shared.down"] = quiet(mat(W, S, 0.8))
                t[p + "mlp.shared.sg"] = mat(1, W, 2.0)
    if overrides:
        for k, v in overrides.items():
            assert t[k].shape == v.shape, k
            t[k] = v
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_model(cfg: dict, model_dir: str, seed: int, overrides: Optional[Dict[str, torch.Tensor]] = None) -> None:
    from safetensors.torch import save_file

    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
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
