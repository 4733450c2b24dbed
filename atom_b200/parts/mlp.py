"""Feed-forwards.  SiLU-gated (atom/models/qwen3.py:166-198, atom/model_ops/activation.py:78-82):
   gu = x W_gate_up^T;  f = silu(gu[:, :I]) * gu[:, I:];  y = f W_down^T.
Dense with the xIELU activation:  y = W_down act(W_up x),
   act(z) = softplus(p) z^2 + z/2 for z > 0,  (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2 otherwise,
with the two numbers (p, q) a parameter of the layer.
GELU-gated:  y = W_down (gelu_tanh(W_gate x) * (W_up x)),  gelu_tanh(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
Dense with the square of relu:  y = W_down relu(W_up x)^2."""
from __future__ import annotations

import math
from typing import Dict

from .. import native
from .base import FeedForward
from .linear import PendingProduct, gated_linear, linear, may_defer
from .registry import register
from .spec import ParamSpec


@register("ffn", "gated_silu")
class GatedSiluMLP(FeedForward):
    graph_safe = True
    takes_scaled_rows = True      # x may be ScaledRows: the first product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the last product on unrun

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

    def params(self) -> Dict[str, ParamSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return {
            "gate_up.weight": ParamSpec((2 * I, H), rows=(I, I)),
            "down.weight": ParamSpec((H, I)),
        }

    def forward(self, x, step, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        f = gated_linear(x, self.w_gate_up_weight, ws.get("ffn.act", (T, self.intermediate_size), dt),
                         lambda m, n: ws.get("ffn.gate_up", (m, n), dt))
        out = ws.get("ffn.out", (T, self.hidden_size), dt)
        if defer and may_defer(f, self.w_down_weight):
            return PendingProduct(f, self.w_down_weight, None, out)
        return linear(f, self.w_down_weight, None, out)


@register("ffn", "gated_gelu")
class GatedGeluMLP(FeedForward):
    graph_safe = True
    takes_scaled_rows = True      # x may be ScaledRows: the first product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the last product on unrun

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

    def params(self) -> Dict[str, ParamSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return {"gate_up.weight": ParamSpec((2 * I, H), rows=(I, I)), "down.weight": ParamSpec((H, I))}

    def forward(self, x, step, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        f = gated_linear(x, self.w_gate_up_weight, ws.get("ffn.act", (T, self.intermediate_size), dt),
                         lambda m, n: ws.get("ffn.gate_up", (m, n), dt), act="gelu_tanh")
        out = ws.get("ffn.out", (T, self.hidden_size), dt)
        if defer and may_defer(f, self.w_down_weight):
            return PendingProduct(f, self.w_down_weight, None, out)
        return linear(f, self.w_down_weight, None, out)


@register("ffn", "dense_xielu")
class DenseXielu(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self._ap = self._aq = 0.0

    def params(self) -> Dict[str, ParamSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return {"up.weight": ParamSpec((I, H)), "down.weight": ParamSpec((H, I)),
                "act": ParamSpec((2,), role="vector", init="normal")}

    def after_load(self) -> None:
        # the activation's two numbers pass through softplus once, in 64-bit, on the host
        p, q = (float(v) for v in self.w_act.double().cpu())
        softplus = lambda v: max(v, 0.0) + math.log1p(math.exp(-abs(v)))
        self._ap, self._aq = softplus(p), softplus(q)

    def forward(self, x, step):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        z = linear(x, self.w_up_weight, None, ws.get("ffn.up", (T, self.intermediate_size), dt))
        native.xielu(z, z, self._ap, self._aq)
        return linear(z, self.w_down_weight, None, ws.get("ffn.out", (T, self.hidden_size), dt))


@register("ffn", "dense_relu2")
class DenseRelu2(FeedForward):
    """y = W_down relu(W_up x)^2."""
    graph_safe = True
    takes_scaled_rows = True      # x may be ScaledRows: the first product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the last product on unrun

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

    def params(self) -> Dict[str, ParamSpec]:
        H, I = self.hidden_size, self.intermediate_size
        return {"up.weight": ParamSpec((I, H)), "down.weight": ParamSpec((H, I))}

    def forward(self, x, step, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        z = linear(x, self.w_up_weight, None, ws.get("ffn.up", (T, self.intermediate_size), dt))
        native.relu2_(z)
        out = ws.get("ffn.out", (T, self.hidden_size), dt)
        if defer and may_defer(z, self.w_down_weight):
            return PendingProduct(z, self.w_down_weight, None, out)
        return linear(z, self.w_down_weight, None, out)
