"""Gated linear attention: a linear-attention mixer with a matrix state per head whose decay depends on the token, one
number per key channel.

   [q | k | v | g | a] = x W^T      q, k (heads x key_dim), v, g (heads x value_dim), a (decay_rank)   one product
   q <- q * key_dim^(-1/2)
   z = W_a2 a + b_a2  (heads x key_dim),   alpha = sigmoid(z)^(1 / tau)
   per head:  S_t = diag(alpha_t) S_(t-1) + k_t v_t^T   from S = 0;    o_t = S_t^T q_t
   y = W_o (concat_h(rmsnorm(o_h; norm, eps)) * silu(g))          the norm runs over one head's columns; its weight
                                                                  [value_dim] is shared by the heads
A request's state is S [heads, key_dim, value_dim] in 32-bit, in its state slot, zero at its first token.  z (the
low-rank product hands it over in 32-bit), the decay, the recurrence and the norm are 32-bit in both precisions.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import native
from .base import Mixer
from .linear import PendingProduct, linear, may_defer
from .registry import register
from .spec import CacheEntry, CacheNeed, ParamSpec


@register("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    graph_safe = True
    takes_scaled_rows = True      # x may be ScaledRows: the projections' product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the output projection on unrun

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay_rank: int, tau: float,
                 norm_eps: float):
        if not tau > 0:
            raise ValueError(f"gated_linear_attention: tau must be positive, got {tau}")
        if torch.cuda.is_available() and not native.gla_supports(key_dim, value_dim):
            raise ValueError(f"gated_linear_attention: key_dim {key_dim} is beyond what the kernel takes (256)")
        self.hidden_size, self.nh, self.dk, self.dv = hidden_size, num_heads, key_dim, value_dim
        self.rank, self.tau, self.norm_eps = decay_rank, float(tau), float(norm_eps)

    def params(self) -> Dict[str, ParamSpec]:
        qk, v = self.nh * self.dk, self.nh * self.dv
        return {"in.weight": ParamSpec((2 * qk + 2 * v + self.rank, self.hidden_size), rows=(qk, qk, v, v, self.rank)),
                "a2.weight": ParamSpec((qk, self.rank)),
                "a2.bias": ParamSpec((qk,), role="vector", init="normal"),
                "norm": ParamSpec((self.dv,), role="vector", init="norm"),
                "o.weight": ParamSpec((self.hidden_size, v))}

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", states=(CacheEntry("S", (self.nh, self.dk, self.dv), "float32"),))

    def forward(self, x, step, cache, writes_cache, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        H, dk, dv = self.nh, self.dk, self.dv
        qk, vv = H * dk, H * dv
        proj = linear(x, self.w_in_weight, None, ws.get("gla.proj", (T, 2 * qk + 2 * vv + self.rank), dt))
        z = linear(proj[:, 2 * qk + 2 * vv:], self.w_a2_weight, None, ws.get("gla.z", (T, qk), torch.float32))
        o = ws.get("gla.o", (T, vv), torch.float32)
        nb, na = native.gla_scratch_elems(T, step.num_seqs, H, dk, dv)
        sb = ws.get("gla.runs", (nb,), torch.float32) if nb else None
        sa = ws.get("gla.decays", (na,), torch.float32) if na else None
        native.gla_scan(o, proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vv], z, self.w_a2_bias, self.tau,
                        dk ** -0.5, cache.states["S"], sb, sa, step.cu_q, step.state_slots, step.num_seqs, H, dk, dv,
                        writes_cache)
        y = ws.get("gla.y", (T, vv), dt)
        native.gla_gate_norm(y, o, proj[:, 2 * qk + vv:2 * qk + 2 * vv], self.w_norm, self.norm_eps, H, dv,
                             step.seq_of_token)
        out = ws.get("gla.out", (T, self.hidden_size), dt)
        if defer and may_defer(y, self.w_o_weight):
            return PendingProduct(y, self.w_o_weight, None, out)
        return linear(y, self.w_o_weight, None, out)
