"""Lightning attention: a linear-attention mixer with a matrix state per head and one constant decay per head.

   [q | k | v | g] = x W^T;   q, k = silu(.) of (heads x key_dim),  v = silu(.) of (heads x value_dim)
   per head:  S_t = decay_h * S_(t-1) + k_t v_t^T   from S = 0;    o_t = S_t^T q_t         (no other scale)
   y = W_o (rmsnorm(concat_h(o); norm, eps) * sigmoid(g))        the norm runs over all heads of a row together
A request's state is S [heads, key_dim, value_dim] in 32-bit, in its state slot, zero at its first token.  The
recurrence, the norm and the gate are 32-bit in both precisions.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import native
from .base import Mixer
from .linear import PendingProduct, linear, may_defer
from .registry import register
from .spec import CacheEntry, CacheNeed, ParamSpec


@register("mixer", "lightning_attention")
class LightningAttention(Mixer):
    graph_safe = True
    takes_scaled_rows = True      # x may be ScaledRows: the projections' product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the output projection on unrun

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay: Sequence[float],
                 norm_eps: float):
        if len(decay) != num_heads:
            raise ValueError(f"lightning_attention: {len(decay)} decays for {num_heads} heads")
        if not native.lightning_supports(key_dim, value_dim):
            raise ValueError(f"lightning_attention: key_dim {key_dim} is beyond what the kernel takes (256)")
        self.hidden_size, self.nh, self.dk, self.dv = hidden_size, num_heads, key_dim, value_dim
        self.decay, self.norm_eps = tuple(float(d) for d in decay), float(norm_eps)
        self._decay_dev: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        qk, v = self.nh * self.dk, self.nh * self.dv
        return {"qkvg.weight": ParamSpec((2 * qk + 2 * v, self.hidden_size), rows=(qk, qk, v, v)),
                "norm": ParamSpec((v,), role="vector", init="norm"),
                "o.weight": ParamSpec((self.hidden_size, v))}

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", states=(CacheEntry("S", (self.nh, self.dk, self.dv), "float32"),))

    def after_load(self) -> None:
        self._decay_dev = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(self.rt.device)

    def forward(self, x, step, cache, writes_cache, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        H, dk, dv = self.nh, self.dk, self.dv
        proj = linear(x, self.w_qkvg_weight, None, ws.get("lt.proj", (T, 2 * H * dk + 2 * H * dv), dt))
        o = ws.get("lt.o", (T, H * dv), torch.float32)
        n = native.lightning_scratch_elems(T, step.num_seqs, H, dk, dv)
        scratch = ws.get("lt.runs", (n,), torch.float32) if n > 1 else None
        native.lightning_scan(o, proj, self._decay_dev, cache.states["S"], scratch, step.cu_q, step.state_slots,
                              step.num_seqs, H, dk, dv, writes_cache)
        y = ws.get("lt.y", (T, H * dv), dt)
        native.lightning_gate_norm(y, o, proj[:, 2 * H * dk + H * dv:], self.w_norm, self.norm_eps, step.seq_of_token)
        out = ws.get("lt.out", (T, self.hidden_size), dt)
        if defer and may_defer(y, self.w_o_weight):
            return PendingProduct(y, self.w_o_weight, None, out)
        return linear(y, self.w_o_weight, None, out)
