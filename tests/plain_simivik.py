"""A plain, slow implementation of the Simivik design in float64 on the CPU: one function per mechanism, whole
sequences at once, no cache, no state carried between calls.  It shares no code with the package; the tests compare
the engine with it.

A model is (config dict as in config.json, {tensor name: float64 tensor}).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, around_zero: bool = False) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps), times w (or 1 + w for a weight stored around zero)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    if w is None:
        return y
    return y * (1.0 + w) if around_zero else y * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), with u = 0 before the first row."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j][None, :]
    return y


def rotate_front(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: the first ``dims`` numbers of every head are rotated by the row's position (pairs
    (i, i + dims/2), angle p * base^(-2i/dims)); the rest pass."""
    if dims == 0:
        return x
    T = x.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = torch.arange(T, dtype=F)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def visible(T: int, size: Optional[int], keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & ((i - j < size) | (j < keep_first))
    return seen


def capped_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    """The attention mixer on h [T, width]; P holds q, k, v, o and (with a convolution) q.conv, k.conv, v.conv."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ P["q"].T, h @ P["k"].T, h @ P["v"].T
    if m.get("conv"):
        q, k, v = short_conv(q, P["q.conv"]), short_conv(k, P["k.conv"]), short_conv(v, P["v.conv"])
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate_front(q, rot["dims"], rot["base"]), rotate_front(k, rot["dims"], rot["base"])
    per = H // G
    k, v = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    mask = m.get("mask")
    seen = visible(T, mask["size"], mask.get("keep_first", 0)) if mask else visible(T, None, 0)
    s = s.masked_fill(~seen[None], -math.inf)
    w = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * dv)
    return o @ P["o"].T


def decayed_state(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float]) -> torch.Tensor:
    """q, k [T, H, d], v [T, H, dv]: S_t = decay_h S_(t-1) + k_t v_t^T from S = 0, o_t = S_t^T q_t; token by token."""
    T, H, d = q.shape
    dv = v.shape[-1]
    lam = torch.tensor(decay, dtype=F)[:, None, None]
    S = torch.zeros(H, d, dv, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = lam * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def lightning(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q, k = silu(h @ P["q"].T).view(T, H, d), silu(h @ P["k"].T).view(T, H, d)
    v = silu(h @ P["v"].T).view(T, H, dv)
    o = decayed_state(q, k, v, m["decay"]).reshape(T, H * dv)
    o = rms_norm(o, P["norm"], eps) * torch.sigmoid(h @ P["g"].T)
    return o @ P["o"].T


def dense_relu2(h: torch.Tensor, P: Dict[str, torch.Tensor]) -> torch.Tensor:
    return torch.relu(h @ P["up"].T) ** 2 @ P["down"].T


def gated_expert(h: torch.Tensor, P: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return (silu(h @ P[prefix + "gate"].T) * (h @ P[prefix + "up"].T)) @ P[prefix + "down"].T


def routed_experts(h: torch.Tensor, P: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    """Every row goes, times its score, INTO its ``top`` experts; a shared expert is added times a gate per row."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.sigmoid(h @ P["router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(s[t], top).indices.tolist():
            out[t] = out[t] + gated_expert((s[t, e] * h[t])[None], P, f"e{e}.")[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ P["shared.sg"].T) * gated_expert(h, P, "shared.")
    return out


def part(W: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def layer(x: torch.Tensor, i: int, cfg: dict, W: Dict[str, torch.Tensor]) -> torch.Tensor:
    L = cfg["layers"][i]
    src = i
    while "weights_of" in cfg["layers"][src]:
        src = cfg["layers"][src]["weights_of"]
    eps = cfg["norm"]["eps"]
    h = rms_norm(x, W[f"l{src}.norm1"], eps, around_zero=True)
    mix = part(W, f"l{src}.mix.")
    if L["type"] == "attention":
        x = x + capped_attention(h, mix, L["mixer"])
    elif L["type"] == "lightning":
        x = x + lightning(h, mix, L["mixer"], eps)
    else:
        raise ValueError(L["type"])
    mlp = L.get("mlp")
    if mlp is not None:
        h = rms_norm(x, W[f"l{src}.norm2"], eps, around_zero=True)
        ff = part(W, f"l{src}.mlp.")
        x = x + (dense_relu2(h, ff) if mlp["kind"] == "dense" else routed_experts(h, ff, mlp))
    return x


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer)."""
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    streams = []
    for i in range(len(cfg["layers"])):
        x = layer(x, i, cfg, W)
        streams.append(x)
    logits = rms_norm(x, W["final.norm"], cfg["norm"]["eps"], around_zero=True) @ W["embed"].T
    return (logits, torch.stack(streams)) if return_layers else logits
