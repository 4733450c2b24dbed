"""Grouped-query attention behind a short causal convolution, with capped scores and a sliding window that always
keeps a request's first tokens.

   [q | k | v] = x W_qkv^T;  q_h, k_g of size key_dim, v_g of size value_dim (they may differ)
   every channel c of q, k and v is convolved over time:  y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]
       (zeros before the request's first token; the request's last taps - 1 projected rows are its state)
   the first rotary_dim numbers of every query and key head are rotated by position * frequency,
       pairs (i, i + rotary_dim / 2); the rest pass
   s[i, j] = scale * q_h[i] . k_g[j];   s <- softcap * tanh(s / softcap)
   position i sees j if j <= i and (i - j < window or j < keep_first); kept tokens keep their positions
   o_h[i] = softmax_j(s[i, j]) v_g[j];   y = concat_h(o_h) W_o^T
Query head h reads kv head h // (num_heads / num_kv_heads).  Convolution, window, kept tokens, cap and rotation are
each an option of the constructor.  The convolution's sums, angles, scores, weights and sums are 32-bit in both
precisions.  The cache keeps pages of k and v (the pages of the first keep_first positions are never given back)
and, with a convolution, the state array ``conv`` [taps - 1, channels].
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


@register("mixer", "conv_window_attention")
class ConvWindowAttention(Mixer):
    graph_safe = True
    takes_scaled_rows = True      # x may be ScaledRows: the qkv product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the output projection on unrun

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 softcap: Optional[float] = None, taps: Optional[int] = None, position: Optional[PartSpec] = None,
                 window: Optional[int] = None, keep_first: int = 0):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if taps is not None and not 1 <= taps <= 64:
            raise ValueError(f"conv_window_attention: {taps} taps are beyond what the kernel takes (1 to 64)")
        if value_dim > 512:
            raise ValueError(f"conv_window_attention: value_dim {value_dim} is beyond what the kernels take (512)")
        self.hidden_size, self.nh, self.nkv, self.dk, self.dv = hidden_size, num_heads, num_kv_heads, key_dim, value_dim
        self.scale, self.softcap, self.taps = float(scale), (float(softcap) if softcap else 0.0), taps
        # (a window beyond any context is one that never closes; the kernels take 32-bit sizes)
        self.window = min(int(window), 1 << 30) if window else None
        self.keep_first = min(int(keep_first), 1 << 30) if window else 0
        self.position = registry.build("position", position) if position is not None else None
        if self.position is not None and not hasattr(self.position, "frequencies"):
            raise ValueError("conv_window_attention rotates by frequencies (a position part with ``frequencies``)")
        if self.position is not None and self.position.rotary_dim > key_dim:
            raise ValueError("rotary_dim exceeds key_dim")
        self.channels = (num_heads + num_kv_heads) * key_dim + num_kv_heads * value_dim

    def params(self) -> Dict[str, ParamSpec]:
        q, k, v = self.nh * self.dk, self.nkv * self.dk, self.nkv * self.dv
        p = {"qkv.weight": ParamSpec((q + k + v, self.hidden_size), rows=(q, k, v)),
             "o.weight": ParamSpec((self.hidden_size, self.nh * self.dv))}
        if self.taps is not None:
            p["conv.weight"] = ParamSpec((q + k + v, self.taps), role="vector", init="half", rows=(q, k, v))
        return p

    def cache_need(self) -> CacheNeed:
        states = ()
        if self.taps is not None and self.taps > 1:
            states = (CacheEntry("conv", (self.taps - 1, self.channels), "compute"),)
        return CacheNeed("pages", window=self.window, keep_first=self.keep_first,
                         entries=(CacheEntry("k", (self.nkv, self.dk)), CacheEntry("v", (self.nkv, self.dv))),
                         states=states)

    def launch_plan(self, step):
        """(into how many shares the tensor-core kernel cuts the key tiles of every unit, or 0 for the plain kernel;
        whether a unit is a token with the query heads of one key head as rows, which steps of single tokens use, or
        a tile of 64 tokens with one head).  Where the units do not fill the device (decoding, short portions) their
        keys are shared out, in shares of at least 128."""
        key = ("conv_window_attention", self.nh, self.nkv, self.dk, self.dv, self.window or 0, self.keep_first)
        plan = step.plans.get(key)
        if plan is None:
            if native.WINDOW_TC and native.window_attention_tc_supports(self.dk, self.dv, self.rt.dtype):
                longest = min(step.max_ctx_len, self.window + self.keep_first) if self.window else step.max_ctx_len
                heads_rows = step.max_q_len <= 1 and self.nh // self.nkv <= native.WINDOW_TC_ROWS
                if heads_rows:
                    units = step.num_tokens * self.nkv
                elif step.max_q_len <= 1:
                    units = step.num_tokens * self.nh
                else:
                    units = (-(-step.num_tokens // native.WINDOW_TC_ROWS) + step.num_seqs - 1) * self.nh
                # (two CTAs fit an SM; steps with prompt portions fill it once before their keys are shared out: the
                # shares cost a pass over 32-bit partial outputs of every row)
                plan = (native.attention_mixed_splits(units, longest, per_sm=2 if step.max_q_len <= 1 else 1,
                                                      min_share=128), heads_rows)
            else:
                plan = (0, False)
            step.plans[key] = plan
        return plan

    def forward(self, x, step, cache, writes_cache, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        nh, nkv, dk, dv = self.nh, self.nkv, self.dk, self.dv
        qkv = linear(x, self.w_qkv_weight, None, ws.get("cwa.qkv", (T, self.channels), dt))
        bt = step.block_tables[cache.group]
        conv_w = self.w_conv_weight if self.taps is not None else None
        conv_state = cache.states.get("conv")
        freq = self.position.frequencies(self.rt) if self.position is not None else None
        q = ws.get("cwa.q", (T, nh * dk), dt)
        native.conv_rope_write(q, qkv, nh, nkv, dk, dv, conv_w, conv_state, freq,
                               self.position.rotary_dim if self.position is not None else 0, step.positions,
                               step.seq_of_token, step.cu_q, step.state_slots, bt, cache.page_size,
                               cache.k_pages if writes_cache else None, cache.v_pages if writes_cache else None,
                               step.status)
        if conv_state is not None and writes_cache:
            native.conv_state_update(conv_state, qkv, step.cu_q, step.state_slots, step.num_seqs)
        o = ws.get("cwa.o", (T, nh * dv), dt)
        nsplit, heads_rows = self.launch_plan(step)
        if nsplit:
            scratch = None
            if nsplit > 1:
                scratch = ws.get("cwa.splits", (native.attention_mixed_scratch_elems(T, nh, dv, nsplit),), torch.float32)
            native.window_attention_tc(o, q, cache.k_pages, cache.v_pages, bt, step.positions, step.seq_of_token,
                                       step.cu_q, step.num_seqs, nh, nkv, dk, dv, self.scale, self.softcap,
                                       self.window or 0, self.keep_first, nsplit, scratch, heads_rows)
        else:
            native.window_attention(o, q, cache.k_pages, cache.v_pages, bt, step.positions, step.seq_of_token, nh, nkv,
                                    dk, dv, self.scale, self.softcap, self.window or 0, self.keep_first)
        out = ws.get("cwa.out", (T, self.hidden_size), dt)
        if defer and may_defer(o, self.w_o_weight):
            return PendingProduct(o, self.w_o_weight, None, out)
        return linear(o, self.w_o_weight, None, out)
