"""A plain, slow implementation of the Kibotar design in float64 on the CPU: one function per mechanism, whole
sequences at once, no cache, no state carried between calls.  It shares no code with the package; the tests compare
the engine with it.

A model is (config dict as in config.json, {tensor name: float64 tensor}).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def embed_tokens(tokens: List[int], table: torch.Tensor, pairs: torch.Tensor, e: dict) -> torch.Tensor:
    """table[token] * scale plus a row of ``pairs`` chosen by (previous token, token); the first token takes the
    last row."""
    big = e["bigram"]
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(big["buckets"] if t == 0 else
                    (tokens[t - 1] * big["mul_prev"] + tok * big["mul_cur"]) % big["buckets"])
    return table[torch.tensor(tokens)] * e["scale"] + pairs[torch.tensor(rows)]


def token_shift(h: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """h_t + (h_(t-1) - h_t) * mu, with zeros before the first row."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (before - h) * mu


def scaled_frequencies(rot: dict) -> torch.Tensor:
    """One frequency per rotated pair; long wavelengths are stretched by ``factor``, short ones kept, and those
    in between blended by where original / wavelength lies between ``low`` and ``high``."""
    dims, base = rot["dims"], rot["base"]
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            lam = 2.0 * math.pi / f
            if lam < sc["original"] / sc["high"]:
                pass
            elif lam > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            else:
                s = (sc["original"] / lam - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=F)


def rotate_front(x: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, d]: the first rot.dims numbers of a head are rotated by the row's position, pair (i, i + dims/2)."""
    if not rot or not rot["dims"]:
        return x
    dims = rot["dims"]
    half = dims // 2
    ang = torch.arange(x.shape[0], dtype=F)[:, None] * scaled_frequencies(rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def gated_linear_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ P["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ P["k"].T).view(T, H, d)
    v = (h @ P["v"].T).view(T, H, dv)
    z = (h @ P["a1"].T) @ P["a2"].T + P["a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o, P["norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ P["g"].T)) @ P["o"].T


def latent_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ P["q"].T).view(T, H, d)
    c = rms_norm(h @ P["dkv"].T, P["dkv.norm"], eps)
    k = (c @ P["uk"].T).view(T, H, d)
    v = (c @ P["uv"].T).view(T, H, dv)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    s = s.masked_fill(~(j <= i)[None], -math.inf)
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhv->ihv", a, v)
    o = o * torch.sigmoid(h @ P["g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ P["o"].T


def pooled_window_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    """Grouped-query attention over the last ``size`` tokens and the means of whole blocks before them, a sink
    of score zero in the denominator, the heads' weights mixed by ``talk``, an output gate."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ P["q"].T + P["q.b"]).view(T, H, d)
    k = (h @ P["k"].T + P["k.b"]).view(T, G, d)
    v = (h @ P["v"].T + P["v.b"]).view(T, G, dv)
    q, k = rotate_front(q, m.get("rot")), rotate_front(k, m.get("rot"))
    mask = m.get("mask")
    size = mask["size"] if mask else None
    pool = mask["pool"] if mask and mask.get("pool") else 0
    nb = T // pool if pool else 0
    if nb:
        k = torch.cat([k, k[:nb * pool].view(nb, pool, G, d).mean(1)], 0)
        v = torch.cat([v, v[:nb * pool].view(nb, pool, G, dv).mean(1)], 0)
    per = H // G
    kk, vv = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]          # [H, T, T + nb]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & (i - j < size)
    if nb:
        b = torch.arange(nb)[None, :]
        seen = torch.cat([seen, b * pool + pool - 1 <= i - size], 1)
    s = s.masked_fill(~seen[None], -math.inf)
    e = torch.exp(s)
    a = e / (1.0 + e.sum(-1, keepdim=True))
    a = torch.einsum("hg,gij->hij", P["talk"], a)
    o = torch.einsum("hij,jhv->ihv", a, vv).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ P["g"].T)
    return o @ P["o"].T + P["o.b"]


def dense_relu2(h: torch.Tensor, P: Dict[str, torch.Tensor]) -> torch.Tensor:
    return torch.relu(h @ P["up"].T) ** 2 @ P["down"].T


def part(W: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def layer(x: torch.Tensor, i: int, cfg: dict, W: Dict[str, torch.Tensor]) -> torch.Tensor:
    L, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}"
    h = token_shift(rms_norm(x, W[f"{p}.norm1"], eps), W[f"{p}.shift"])
    mix = part(W, f"{p}.mix.")
    if L["type"] == "gla":
        y = gated_linear_attention(h, mix, L["mixer"], eps)
    elif L["type"] == "latent_attention":
        y = latent_attention(h, mix, L["mixer"], eps)
    elif L["type"] == "attention":
        y = pooled_window_attention(h, mix, L["mixer"])
    else:
        raise ValueError(L["type"])
    x = x + rms_norm(y, W[f"{p}.norm1b"], eps)
    if L.get("mlp") is not None:
        y = dense_relu2(rms_norm(x, W[f"{p}.norm2"], eps), part(W, f"{p}.mlp."))
        x = x + rms_norm(y, W[f"{p}.norm2b"], eps)
    return x


def run_order(cfg: dict):
    """(layer, number of the pass or None) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        out += [(i, t) for i in range(loop["start"], loop["stop"])]
    return out + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens, return_layers: bool = False):
    """Logits [T, vocab] of one sequence from its first token."""
    x = embed_tokens(list(tokens), W["embed"], W["bigram"], cfg["embedding"])
    after = []
    loop = cfg.get("loop")
    for i, t in run_order(cfg):
        if t is not None and i == loop["start"]:
            x = x + W["loop.step"][t]
        x = layer(x, i, cfg, W)
        after.append(x)
    logits = rms_norm(x, W["final.norm"], cfg["norm"]["eps"]) @ W["embed"].T
    return (logits, after) if return_layers else logits
