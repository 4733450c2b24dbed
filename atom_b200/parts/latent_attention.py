"""Attention through a latent: a token's keys and values are linear maps of one small normalised vector, which is
all the cache keeps of it, beside a short rotated key part that every head shares.

   [dq | dkv | g] = W_in h                              one product; dkv absent when another layer's cache is read
   cq = rmsnorm(dq; w_dq),   q_h = W_uq,h cq = [qn_h (dim) | qr_h (rot_dim)],   qr_h rotated
   c = rmsnorm(dkv[:kv_rank]; w_dkv),   kr = rotated dkv[kv_rank:]              the cached row is [c | kr]
   s_h[i, j] = scale * (qn_h[i] . (W_uk,h c[j]) + qr_h[i] . kr[j])              0 <= i - j < window
   a_h[i, j] = exp(s_h[i, j]) / (exp(sink_h) + sum_j' exp(s_h[i, j']))         (no sink term without sink)
   y = W_o (concat_h(W_uv,h sum_j a_h[i, j] c[j]) * sigmoid(g))                 (no gate without gate)
The key map is folded into the query, qn_h . (W_uk,h c) = (W_uk,h^T qn_h) . c, and the value map is applied after
the weighted sum, so the attention kernel reads one row of kv_rank + rot_dim numbers per key for all heads and the
keys and values of cached tokens are never rebuilt.  Rotation: the first ``rot_dims`` numbers of the rotated parts,
pair (i, i + rot_dims/2), by the frequencies and the magnitude of the position part (parts/rope.py).

Options: ``q_rank`` None leaves the query latent out (q_h = W_q h directly: the first rows of the stacked product, no
norm, no W_uq); ``rot_dim`` 0 with ``position`` None leaves the rotated part out; ``gate`` "head" gates a head's
output with ONE number, sigmoid(W_g h)_h, with W_g of ``heads`` rows.

A layer with ``reads_cache_of_other`` has no W_dkv: the run entry gives it the cache slot of the layer whose rows it
reads (written earlier in the same step), with maps, queries, window, sink and gate of its own.  ``cache_window``
is the window the cache has to keep for all its readers (None: every row).
Folded queries, angles, scores, weights and sums are 32-bit in both precisions.
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


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True
    takes_scaled_rows = True      # x may be ScaledRows: the stacked first product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the output projection on unrun

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int,
                 q_rank: Optional[int], kv_rank: int, scale: float, norm_eps: float, position: Optional[PartSpec],
                 window: Optional[int] = None, cache_window: Optional[int] = None, sink: bool = False, gate=False,
                 reads_cache_of_other: bool = False):
        if gate not in (False, True, "head"):
            raise ValueError(f"latent_attention: gate is False, True or 'head', got {gate!r}")
        if position is None:
            if rot_dim:
                raise ValueError("latent_attention: a rotated part needs a position encoding")
            position = PartSpec("none")
        self.hidden_size, self.nh, self.dn, self.rd, self.dv = hidden_size, num_heads, head_dim, rot_dim, value_dim
        self.q_rank, self.R, self.scale, self.norm_eps = q_rank, kv_rank, float(scale), norm_eps
        self.window, self.cache_window = window, cache_window
        self.sink, self.gate, self.borrows = sink, gate, reads_cache_of_other
        self.position = registry.build("position", position)
        if self.position.rotary_dim > rot_dim:
            raise ValueError(f"latent_attention: {self.position.rotary_dim} rotated numbers in a part of {rot_dim}")
        if window is not None and (cache_window is not None and cache_window < window):
            raise ValueError("latent_attention: the cache keeps fewer rows than the window looks back")
        if not native_supports(num_heads, kv_rank, rot_dim):
            raise ValueError(f"latent_attention: kv_rank {kv_rank} + rot_dim {rot_dim} is beyond what the kernel takes")
        self._sink = self._ukT = self._uv = self._freq = None

    def _in_rows(self):
        rows = [self.q_rank if self.q_rank is not None else self.nh * (self.dn + self.rd)]
        if not self.borrows:
            rows.append(self.R + self.rd)
        if self.gate:
            rows.append(self.nh if self.gate == "head" else self.nh * self.dv)
        return tuple(rows)

    def params(self) -> Dict[str, ParamSpec]:
        H, W = self.nh, self.hidden_size
        rows = self._in_rows()
        p = {
            "in.weight": ParamSpec((sum(rows), W), rows=rows),
            "uk.weight": ParamSpec((H * self.dn, self.R)),
            "uv.weight": ParamSpec((H * self.dv, self.R)),
            "o.weight": ParamSpec((W, H * self.dv)),
        }
        if self.q_rank is not None:
            p["dq.norm"] = ParamSpec((self.q_rank,), role="vector", init="norm")
            p["uq.weight"] = ParamSpec((H * (self.dn + self.rd), self.q_rank))
        if not self.borrows:
            p["dkv.norm"] = ParamSpec((self.R,), role="vector", init="norm")
        if self.sink:
            p["sink"] = ParamSpec((H,), role="vector", init="normal")
        return p

    def cache_need(self) -> CacheNeed:
        return CacheNeed("pages", window=self.cache_window, entries=(CacheEntry("latent", (self.R + self.rd,)),))

    def after_load(self) -> None:
        H = self.nh
        self._sink = self.w_sink.float().contiguous() if self.sink else None
        # W_uk,h^T as the matrix of the folded query's product: [H, kv_rank, dim]
        self._ukT = self.w_uk_weight.view(H, self.dn, self.R).transpose(1, 2).contiguous()
        self._uv = self.w_uv_weight.view(H, self.dv, self.R)
        self._freq = self.position.frequencies(self.rt) if self.rd else None

    def launch_plan(self, step):
        """(query rows of a tensor-core tile, or 0 for the plain kernel; into how many shares every unit's keys are
        cut).  The tensor-core kernel's unit is a tile of a few consecutive tokens of a request with a group of heads:
        64 rows in steps with prompt portions, 16 in steps of single tokens; the plain kernel's is a token with a group
        of heads.  Where the units do not fill the device (decoding, short portions) their keys are shared out."""
        key = ("latent_attention", self.nh, self.R, self.rd, self.window or 0)
        plan = step.plans.get(key)
        if plan is None:
            longest = min(step.max_ctx_len, self.window) if self.window else step.max_ctx_len
            if native.LATENT_TC and native.latent_attention_tc_supports(self.nh, self.R, self.rd, self.rt.dtype):
                rows = 16 if step.max_q_len <= 1 else 64
                per_tile = native.latent_attention_tc_tile_tokens(self.nh, rows)
                tiles = step.num_tokens if step.max_q_len <= 1 else -(-step.num_tokens // per_tile) + step.num_seqs - 1
                units, per_sm, share = tiles * -(-self.nh // rows), (2 if rows == 16 else 1), (32 if rows == 16 else 64)
            else:
                rows, per_sm, share = 0, 2, 64
                units = step.num_tokens * -(-self.nh // native.latent_attention_head_group(self.nh, self.R, self.rd))
            plan = step.plans[key] = (rows, native.attention_mixed_splits(units, longest, per_sm=per_sm, min_share=share))
        return plan

    def forward(self, x, step, cache, writes_cache, defer=False):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        H, dn, rd, dv, R, Rq = self.nh, self.dn, self.rd, self.dv, self.R, self.q_rank
        rows = self._in_rows()
        proj = linear(x, self.w_in_weight, None, ws.get("lat.in", (T, sum(rows)), dt))
        bt = step.block_tables[cache.group]
        pages = cache.pages["latent"]
        pos = self.position
        mag = getattr(pos, "magnitude", 1.0)
        direct = Rq is None         # the queries are the stacked product's first rows as they are
        cq = None if direct else ws.get("lat.cq", (T, Rq), dt)
        wq = None if direct else self.w_dq_norm
        if self.borrows or not writes_cache:
            if not direct:
                native.latent_prepare(cq, proj, 0, wq, self.norm_eps, step.positions, step.seq_of_token)
        else:
            native.latent_prepare(cq, proj, 0, wq, self.norm_eps, step.positions, step.seq_of_token,
                                  kv_off=rows[0], kv_rank=R, rot_dim=rd, rot_dims=pos.rotary_dim, wkv=self.w_dkv_norm,
                                  freq=self._freq, mag=mag, block_table=bt, page_size=cache.page_size,
                                  pages=pages, status=step.status)
        if direct:
            q = proj[:, :rows[0]].view(T, H, dn + rd) if proj.stride(0) == rows[0] else \
                proj.as_strided((T, H, dn + rd), (proj.stride(0), dn + rd, 1))
        else:
            q = linear(cq, self.w_uq_weight, None, ws.get("lat.q", (T, H * (dn + rd)), dt)).view(T, H, dn + rd)
        qf = ws.get("lat.qf", (T, H, R + rd), torch.float32)
        native.gemm_batched(qf[:, :, :R], q[:, :, :dn], self._ukT)
        if rd:
            native.rotate_pairs(qf, R, q, dn, rd, pos.rotary_dim, self._freq, mag, step.positions, step.seq_of_token)
        olat = ws.get("lat.olat", (T, H, R), dt)
        tile_rows, nsplit = self.launch_plan(step)
        scratch = None
        if nsplit > 1:
            scratch = ws.get("lat.splits", (native.latent_attention_scratch_elems(T, H, R, nsplit),), torch.float32)
        if tile_rows:
            native.latent_attention_tc(olat, qf, pages, bt, step.positions, step.cu_q, step.num_seqs, R, rd, self.scale,
                                       self.window or 0, self._sink, nsplit, scratch, step.seq_of_token, tile_rows)
        else:
            native.latent_attention(olat, qf, pages, bt, step.positions, step.seq_of_token, R, rd, self.scale,
                                    self.window or 0, self._sink, nsplit, scratch)
        heads = ws.get("lat.heads", (T, H, dv), dt)
        native.gemm_batched(heads, olat, self._uv)
        heads = heads.view(T, H * dv)
        if self.gate == "head":
            native.head_gate(heads.view(T, H, dv), proj[:, sum(rows) - H:])
        elif self.gate:
            g_off = sum(rows) - H * dv
            native.sigmoid_mul(heads, proj[:, g_off:])
        out = ws.get("lat.out", (T, self.hidden_size), dt)
        if defer and may_defer(heads, self.w_o_weight):
            return PendingProduct(heads, self.w_o_weight, None, out)
        return linear(heads, self.w_o_weight, None, out)


def native_supports(heads: int, kv_rank: int, rot_dim: int) -> bool:
    """Sizes the attention kernel takes; asked without loading the library where there is no device."""
    if not torch.cuda.is_available():
        return heads > 0 and kv_rank > 0 and rot_dim >= 0
    return native.latent_attention_supports(heads, kv_rank, rot_dim)
