"""Token embedding (atom/model_ops/embed_head.py:177) and output head (:249-252).

The embedding writes the 32-bit residual stream (times a constant ``scale`` where a model has one); the head multiplies the normalised rows
whose logits are wanted by the output matrix and returns 32-bit logits.  A tied head uses
the embedding's table (atom/models/qwen3.py:339-340)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import native
from .base import Part
from .linear import linear
from .registry import register
from .spec import CacheEntry, CacheNeed, ParamSpec


@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0):
        self.vocab_size, self.hidden_size, self.scale = vocab_size, hidden_size, float(scale)

    def params(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def forward(self, token_ids: torch.Tensor, T: int) -> torch.Tensor:
        out = self.rt.workspace.get("residual", (T, self.hidden_size), torch.float32)
        native.embedding(out, self.w_weight, token_ids, self.scale)
        return out


@register("embedding", "pair_embedding")
class PairEmbedding(Part):
    """x = weight[token] * scale + pairs[(previous token * mul_prev + token * mul_cur) mod buckets]; a request's first
    token takes the last row of ``pairs`` ([buckets + 1, hidden]).  The previous token is part of a request's state (one
    int32 in its state slot), so the embedding declares a cache need as a mixer does and ``forward`` takes the step
    and the view of its cache slot."""
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int, scale: float = 1.0):
        if buckets <= 0 or mul_prev < 0 or mul_cur < 0:
            raise ValueError("pair_embedding: buckets must be positive and the multipliers not negative")
        self.vocab_size, self.hidden_size, self.scale = vocab_size, hidden_size, float(scale)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)

    def params(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size)),
                "pairs": ParamSpec((self.buckets + 1, self.hidden_size))}

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed("state", states=(CacheEntry("previous", (1,), "int32"),))

    def forward(self, token_ids: torch.Tensor, T: int, step=None, cache=None) -> torch.Tensor:
        out = self.rt.workspace.get("residual", (T, self.hidden_size), torch.float32)
        native.pair_embedding(out, self.w_weight, self.w_pairs, token_ids, step.positions, step.seq_of_token, step.cu_q,
                              step.state_slots, cache.states["previous"], self.buckets, self.mul_prev, self.mul_cur,
                              self.scale)
        return out


@register("stream", "step_vectors")
class StepVectors(Part):
    """Vectors of the residual stream's width that run entries add to it (``RunEntry.add_step`` names the row): a
    design that runs a span of its layers several times marks every pass with one."""
    graph_safe = True

    def __init__(self, count: int, hidden_size: int):
        self.count, self.hidden_size = count, hidden_size

    def params(self) -> Dict[str, ParamSpec]:
        return {"table": ParamSpec((self.count, self.hidden_size), role="vector", init="normal")}

    def add(self, residual: torch.Tensor, row: int) -> None:
        native.add_row(residual, self.w_table[row])


@register("head", "lm_head")
class LMHead(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool):
        self.vocab_size, self.hidden_size, self.tied = vocab_size, hidden_size, tied

    def params(self) -> Dict[str, ParamSpec]:
        if self.tied:
            return {}
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def tie(self, embedding: TokenEmbedding) -> None:
        self.w_weight = embedding.w_weight

    def forward(self, x: torch.Tensor, out=None) -> torch.Tensor:
        """x: [R, hidden] -> logits [R, vocab] float32; into ``out`` if given, else a fresh
        tensor the caller may keep."""
        if out is None:
            out = torch.empty((x.shape[0], self.vocab_size), dtype=torch.float32, device=x.device)
        return linear(x, self.w_weight, None, out[: x.shape[0]])
