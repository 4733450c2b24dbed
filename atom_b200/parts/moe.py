"""Routed experts: a mixture of small gated feed-forwards of which every row uses ``top``.

   z = W_router x  (32-bit);   score = sigmoid(z)  or  softmax(z)            ``score``
   the ``top`` experts with the largest scores are chosen (ties: the lower index); their weights are their scores,
       divided by their sum if ``renormalize``
   expert e:  f_e(h) = W_down,e (silu(W_gate,e h) * (W_up,e h))
   y = sum over the chosen e of  f_e(w_e * x)   (``weight_on`` "input")   or   w_e * f_e(x)   ("output")
   with a shared expert of ``shared_size``:  y += sigmoid(w_sg . x) * f_shared(x)   (``shared_gate``; without it the
       shared expert is added as it is)
Router logits, scores, weights and the gate are 32-bit in both precisions.  Rows are sorted by expert on the device
(no host round trip: the launches depend on the step's shape alone), every expert's rows run as tiles of one grouped
product, and a row's choices are added up in a fixed order.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import native
from .base import FeedForward
from .linear import gated_linear, linear
from .registry import register
from .spec import ParamSpec


@register("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, num_experts: int, top: int, intermediate_size: int,
                 shared_size: Optional[int] = None, score: str = "sigmoid", renormalize: bool = False,
                 weight_on: str = "input", shared_gate: bool = False):
        if score not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError(f"routed_experts: score {score!r} / weight_on {weight_on!r} not known")
        if not 1 <= top <= min(num_experts, 32) or num_experts > 1024:
            raise ValueError(f"routed_experts: top {top} of {num_experts} experts is beyond what the kernels take")
        self.hidden_size, self.E, self.top, self.ff = hidden_size, num_experts, top, intermediate_size
        self.shared_size = shared_size or None
        self.score, self.renormalize, self.weight_on = score, bool(renormalize), weight_on
        self.shared_gate = bool(shared_gate) and self.shared_size is not None

    def params(self) -> Dict[str, ParamSpec]:
        H, E, F = self.hidden_size, self.E, self.ff
        rows = (E, 1) if self.shared_gate else (E,)
        p = {"router.weight": ParamSpec((sum(rows), H), rows=rows),
             "gate_up.weight": ParamSpec((E * 2 * F, H), rows=(F,) * (2 * E)),
             "down.weight": ParamSpec((E * H, F), rows=(H,) * E)}
        if self.shared_size is not None:
            S = self.shared_size
            p["shared.gate_up.weight"] = ParamSpec((2 * S, H), rows=(S, S))
            p["shared.down.weight"] = ParamSpec((H, S))
        return p

    def forward(self, x, step):
        T, H = x.shape
        E, top, F = self.E, self.top, self.ff
        ws, dt = self.rt.workspace, self.rt.dtype
        R = T * top
        n_logits = self.w_router_weight.shape[0]
        logits = linear(x, self.w_router_weight, None, ws.get("moe.logits", (T, n_logits), torch.float32))
        ids = ws.get("moe.ids", (T, top), torch.int32)
        wts = ws.get("moe.wts", (T, top), torch.float32)
        counts = ws.get("moe.counts", (1024,), torch.int32, zero=True)     # zero between steps: moe_place leaves it so
        native.moe_route(logits, E, top, self.score, self.renormalize, step.seq_of_token, ids, wts, counts)
        offsets = ws.get("moe.offsets", (E + 1,), torch.int32)
        row_token = ws.get("moe.row_token", (R,), torch.int32)
        row_w = ws.get("moe.row_w", (R,), torch.float32)
        pair_pos = ws.get("moe.pair_pos", (R,), torch.int32)
        native.moe_place(ids, wts, E, counts, offsets, row_token, row_w, pair_pos)
        on_input = self.weight_on == "input"
        if not on_input:
            ones = ws.get("moe.ones", (R,), torch.float32)
            ones.fill_(1.0)
        act = ws.get("moe.act", (R, F), dt)
        native.moe_gemm(act, x, self.w_gate_up_weight.view(E, 2 * F, H), offsets, gated=True, row_token=row_token,
                        row_w=row_w if on_input else ones)
        y = ws.get("moe.y", (R, H), dt)
        native.moe_gemm(y, act, self.w_down_weight.view(E, H, F), offsets)
        shared = None
        if self.shared_size is not None:
            S = self.shared_size
            f = gated_linear(x, self.w_shared_gate_up_weight, ws.get("moe.shared.act", (T, S), dt),
                             lambda m, n: ws.get("moe.shared.gate_up", (m, n), dt))
            shared = linear(f, self.w_shared_down_weight, None, ws.get("moe.shared.out", (T, H), dt))
        out = ws.get("moe.out", (T, H), dt)
        native.moe_combine(out, y, pair_pos, top, None if on_input else wts, shared,
                           logits[:, E:E + 1] if self.shared_gate else None, step.seq_of_token)
        return out
