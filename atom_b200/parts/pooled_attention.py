"""Grouped-query attention over a sliding window and, before the window, one pooled key and value per whole block of
tokens; the softmax may hold a sink of score zero, the heads' weights may be mixed after the softmax, the output may
pass a gate.

   q, k, v = W_q h (+ b_q), W_k h (+ b_k), W_v h (+ b_v)      one stacked product (with the gate's rows when there is one)
   the first ``position.rotary_dim`` numbers of every query and key head are rotated (pairs (i, i + dims/2), angle
   position * frequency, the frequencies from the position part); the rest pass
   token j is seen from position i if 0 <= i - j < window; block b (positions b pool .. b pool + pool - 1) if
   b pool + pool - 1 <= i - window: its key is the mean of the block's keys as the cache holds them, its value the mean
   of the block's values; tokens that have left the window and whose block is not yet seen are not seen at all
   p_h[x] = exp(scale q_h.k[x]) / (sink + sum_x' exp(scale q_h.k[x']))    over the seen tokens and blocks together,
            sink = 1 with ``zero_sink`` (a sink of score zero that has no value), else 0
   w_h = sum_g talk[h, g] p_g  (with ``talk``; the sink's share is not mixed);   o_h = sum_x w_h[x] v_kv(h)[x]
   y = W_o (concat_h(o_h) * sigmoid(W_g h)) (+ b_o)                          (no gate without ``gate``)
The cache keeps, per token, key and value of the last max(window, pool) positions in pages, and per whole block one
pooled key and value in pages of a second group that the window never gives back (``CacheNeed.block_entries``).
Without a window every earlier token is seen and nothing is pooled.  Angles, scores, weights, the mixing and the sums are
32-bit in both precisions.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import native
from . import registry
from .base import Mixer
from .linear import PendingProduct, linear, may_defer
from .registry import register
from .spec import CacheEntry, CacheNeed, ParamSpec, PartSpec


@register("mixer", "pooled_window_attention")
class PooledWindowAttention(Mixer):
    graph_safe = True
    takes_scaled_rows = True
    defers_output = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 position: Optional[PartSpec] = None, window: Optional[int] = None, pool: Optional[int] = None,
                 zero_sink: bool = False, talk: bool = False, gate: bool = False, bias: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError("pooled_window_attention: heads must be a multiple of kv heads")
        if pool and not window:
            raise ValueError("pooled_window_attention: blocks are pooled only before a window")
        if torch.cuda.is_available() and not native.pooled_attention_supports(num_heads, num_kv_heads, key_dim, value_dim):
            raise ValueError(f"pooled_window_attention: {num_heads} heads of value size {value_dim} are beyond what "
                             "the kernel takes")
        self.hidden_size, self.nh, self.nkv, self.dk, self.dv = hidden_size, num_heads, num_kv_heads, key_dim, value_dim
        self.scale, self.window, self.pool = float(scale), window or None, pool or None
        self.zero_sink, self.talk, self.gate, self.bias = bool(zero_sink), bool(talk), bool(gate), bool(bias)
        self.position = registry.build("position", position) if position is not None else None
        if self.position is not None and self.position.rotary_dim > key_dim:
            raise ValueError("pooled_window_attention: more rotated numbers than a key has")
        self._talk = None

    def _rows(self):
        rows = [self.nh * self.dk, self.nkv * self.dk, self.nkv * self.dv]
        if self.gate:
            rows.append(self.nh * self.dv)
        return tuple(rows)

    def params(self) -> Dict[str, ParamSpec]:
        rows = self._rows()
        p = {"in.weight": ParamSpec((sum(rows), self.hidden_size), rows=rows),
             "o.weight": ParamSpec((self.hidden_size, self.nh * self.dv))}
        if self.bias:
            # (a gate has no bias: its rows of the stacked bias are zeros, made after loading)
            p["qkv.bias"] = ParamSpec((sum(rows[:3]),), role="vector", init="normal", rows=rows[:3])
            p["o.bias"] = ParamSpec((self.hidden_size,), role="vector", init="normal")
        if self.talk:
            p["talk"] = ParamSpec((self.nh, self.nh), role="vector", init="eye")
        return p

    def cache_need(self) -> CacheNeed:
        entries = (CacheEntry("k", (self.nkv, self.dk)), CacheEntry("v", (self.nkv, self.dv)))
        if self.window is None:
            return CacheNeed("pages", entries=entries)
        if self.pool is None:
            return CacheNeed("pages", window=self.window, entries=entries)
        # a block's rows are read once more when its last token arrives: the cache keeps a block's length at least
        return CacheNeed("pages", window=max(self.window, self.pool), entries=entries, block=self.pool,
                         block_entries=(CacheEntry("pk", (self.nkv, self.dk)), CacheEntry("pv", (self.nkv, self.dv))))

    def after_load(self) -> None:
        self._talk = self.w_talk.float().contiguous() if self.talk else None
        self._in_bias = None
        if self.bias:
            b = self.w_qkv_bias
            if self.gate:
                b = torch.cat([b, torch.zeros(self.nh * self.dv, dtype=b.dtype, device=b.device)])
            self._in_bias = b.contiguous()

    def launch_plan(self, step):
        """("split", shares) for steps of few tokens: every token's keys are shared out among CTAs; ("tiles", 0) for the
        tensor-core kernel's tiles of 16 tokens; ("tokens", 0) for the plain kernel, a CTA a token."""
        key = ("pooled_window_attention", self.nh, self.nkv, self.dk, self.dv, self.window or 0, self.pool or 0)
        plan = step.plans.get(key)
        if plan is None:
            T = step.num_tokens
            if native.POOLED_SPLIT_ROWS and T <= native.POOLED_SPLIT_ROWS and \
                    native.pooled_attention_split_supports(self.nh, self.nkv, self.dk, self.dv):
                longest = min(step.max_ctx_len, self.window) if self.window else step.max_ctx_len
                if self.pool:
                    longest += step.max_ctx_len // self.pool
                plan = ("split", native.pooled_attention_splits(T, max(longest, 1)))
            elif native.POOLED_TC and native.pooled_attention_tc_supports(self.nh, self.nkv, self.dk, self.dv, self.rt.dtype):
                plan = ("tiles", 0)
            else:
                plan = ("tokens", 0)
            step.plans[key] = plan
        return plan

    def forward(self, x, step, cache, writes_cache, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        nh, nkv, dk, dv = self.nh, self.nkv, self.dk, self.dv
        rows = self._rows()
        proj = linear(x, self.w_in_weight, self._in_bias, ws.get("pwa.in", (T, sum(rows)), dt))
        bt = step.block_tables[cache.group]
        pos = self.position
        freq = pos.frequencies(self.rt) if pos is not None and pos.rotary_dim else None
        q = ws.get("pwa.q", (T, nh * dk), dt)
        native.conv_rope_write(q, proj, nh, nkv, dk, dv, None, None, freq, pos.rotary_dim if freq is not None else 0,
                               step.positions, step.seq_of_token, step.cu_q, step.state_slots, bt, cache.page_size,
                               cache.k_pages if writes_cache else None, cache.v_pages if writes_cache else None,
                               step.status)
        pk = pv = pool_bt = None
        if self.pool is not None:
            pk, pv = cache.block_pages["pk"], cache.block_pages["pv"]
            pool_bt = step.block_tables[cache.block_group]
            if writes_cache:
                native.pool_blocks(cache.k_pages, cache.v_pages, pk, pv, bt, pool_bt, cache.page_size, step.positions,
                                   step.seq_of_token, T, self.pool, step.status)
        o = ws.get("pwa.o", (T, nh * dv), dt)
        gate = proj[:, sum(rows[:3]):] if self.gate else None
        how, nsplit = self.launch_plan(step)
        if how == "split":
            scratch = ws.get("pwa.shares", (native.pooled_attention_scratch_elems(T, nh, nkv, dv, nsplit),), torch.float32)
            native.pooled_attention_split(o, scratch, q, cache.k_pages, cache.v_pages, pk, pv, bt, pool_bt, cache.page_size,
                                          step.positions, step.seq_of_token, nh, self.scale, self.window or 0,
                                          self.pool or 0, self.zero_sink, self._talk, gate, nsplit)
        elif how == "tiles":
            native.pooled_attention_tc(o, q, cache.k_pages, cache.v_pages, pk, pv, bt, pool_bt, cache.page_size,
                                       step.positions, step.cu_q, step.num_seqs, nh, self.scale, self.window or 0,
                                       self.pool or 0, self.zero_sink, self._talk, gate)
        else:
            native.pooled_attention(o, q, cache.k_pages, cache.v_pages, pk, pv, bt, pool_bt, cache.page_size,
                                    step.positions, step.seq_of_token, nh, self.scale, self.window or 0, self.pool or 0,
                                    self.zero_sink, self._talk, gate)
        out = ws.get("pwa.out", (T, self.hidden_size), dt)
        bias = self.w_o_bias if self.bias else None
        if defer and bias is None and may_defer(o, self.w_o_weight):
            return PendingProduct(o, self.w_o_weight, None, out)
        return linear(o, self.w_o_weight, bias, out)
