"""Arrangements of a layer's parts around the residual stream.

An arrangement declares the parts it is put together from: ``slots`` maps each part's name in
the layer to its category in the registries (the model builds exactly these from the layer's
spec and hands them to the constructor by name); names listed in ``optional`` may be left out
of a layer.  The part named ``mixer``, if there is one, is the one whose cache the run entry's
cache slot holds.

"prenorm" is the one of atom/models/qwen3.py:248-258: the residual is a running 32-bit
sum; each sub-block's output is added to it inside the next norm's kernel:
   r += delta;  a = norm1(r);  m = mixer(a);  r += m;  b = norm2(r);  delta' = ffn(b).

"prenorm_scaled" is "prenorm" with every sub-block's output entering the residual times a constant m, and with
the feed-forward (and its norm) optional:
   r += m * delta;  a = norm1(r);  x = mixer(a);  [r += m * x;  b = norm2(r);  x = ffn(b)]  -> x, added times m
by whoever comes next (``delta_scale`` tells the model the factor of what ``run`` returned).

"parallel" has one norm whose output both the mixer and the feed-forward read, and adds both to the residual:
   r += delta;  h = norm(r);  r += mixer(h) + ffn(h)        (a layer may have no feed-forward).

"sandwich" puts a norm before and after each sub-block (the feed-forward and its two norms optional):
   r += delta;  a = norm1(r);  r += norm1b(mixer(a));  [b = norm2(r);  r += norm2b(ffn(b))]
A sub-block's output travels to the next norm as a ``NormedDelta``, so that the norm after a sub-block, the add and
the norm before the next sub-block are one kernel.

Between parts that say they can, an output travels as a product still to run and normalised rows
as ``ScaledRows`` (parts/linear.py), so that in a step of few rows the norms need no kernel of their
own; a part that says nothing gets and gives plain tensors.
"""
from __future__ import annotations

from .. import native
from .linear import NormedDelta, resolve
from .registry import register


def _add_norm(norm, residual, delta, tag, receiver, **kw):
    if getattr(norm, "fuses_products", False):
        return norm.add_norm(residual, delta, tag, scaled_ok=getattr(receiver, "takes_scaled_rows", False), **kw)
    return norm.add_norm(residual, resolve(delta), tag, **kw)


def _forward(part, *args):
    if getattr(part, "defers_output", False):
        return part.forward(*args, defer=True)
    return part.forward(*args)


@register("arrangement", "prenorm")
class PreNormBlock:
    slots = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "ffn"}
    optional = ()
    takes_pending = True      # delta may be a PendingProduct, and so may what run() returns

    def __init__(self, mixer_norm, mixer, ffn_norm, ffn):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def run(self, residual, delta, step, cache, writes_cache):
        """residual: [T, hidden] float32, updated in place.  delta: the previous block's output
        (None for the first).  Returns this block's output, to be added by the next norm."""
        a = _add_norm(self.mixer_norm, residual, delta, "norm.mixer", self.mixer)
        m = _forward(self.mixer, a, step, cache, writes_cache)
        b = _add_norm(self.ffn_norm, residual, m, "norm.ffn", self.ffn)
        return _forward(self.ffn, b, step)


@register("arrangement", "prenorm_scaled")
class ScaledPreNormBlock:
    slots = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "ffn"}
    optional = ("ffn_norm", "ffn")
    takes_pending = True      # delta may be a PendingProduct, and so may what run() returns

    def __init__(self, mixer_norm, mixer, ffn_norm=None, ffn=None, residual_mult: float = 1.0):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("prenorm_scaled: a feed-forward and its norm come together")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.delta_scale = float(residual_mult)     # the factor of the output that run() hands on

    def run(self, residual, delta, step, cache, writes_cache, delta_scale=None):
        """delta_scale: the factor of the incoming delta (the block's own constant unless the model says otherwise)."""
        m = self.delta_scale
        a = _add_norm(self.mixer_norm, residual, delta, "norm.mixer", self.mixer,
                      delta_scale=m if delta_scale is None else delta_scale)
        x = _forward(self.mixer, a, step, cache, writes_cache)
        if self.ffn is None:
            return x
        b = _add_norm(self.ffn_norm, residual, x, "norm.ffn", self.ffn, delta_scale=m)
        return _forward(self.ffn, b, step)


@register("arrangement", "sandwich")
class SandwichBlock:
    slots = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm", "ffn_norm": "norm", "ffn": "ffn",
             "ffn_post_norm": "norm"}
    optional = ("ffn_norm", "ffn", "ffn_post_norm")
    takes_pending = True      # delta may be a NormedDelta (or a PendingProduct), and run() returns a NormedDelta

    def __init__(self, mixer_norm, mixer, mixer_post_norm, ffn_norm=None, ffn=None, ffn_post_norm=None):
        if len({ffn is None, ffn_norm is None, ffn_post_norm is None}) != 1:
            raise ValueError("sandwich: a feed-forward and its two norms come together")
        for n in (mixer_post_norm, ffn_post_norm):
            if n is not None and getattr(n, "weight_offset", 0.0):
                raise ValueError("sandwich: the norms after a sub-block take plain weights")
        self.mixer_norm, self.mixer, self.mixer_post_norm = mixer_norm, mixer, mixer_post_norm
        self.ffn_norm, self.ffn, self.ffn_post_norm = ffn_norm, ffn, ffn_post_norm

    @staticmethod
    def _normed(x, norm, tag):
        out = norm.rt.workspace.get(tag, tuple(x.shape), x.dtype)
        return NormedDelta(x, norm.w_weight, norm.eps, out)

    def run(self, residual, delta, step, cache, writes_cache):
        a = self.mixer_norm.add_norm(residual, delta, "norm.mixer")
        m = self.mixer.forward(a, step, cache, writes_cache)
        m = self._normed(m, self.mixer_post_norm, "norm.mixer.post")
        if self.ffn is None:
            return m
        b = self.ffn_norm.add_norm(residual, m, "norm.ffn")
        f = self.ffn.forward(b, step)
        return self._normed(f, self.ffn_post_norm, "norm.ffn.post")


@register("arrangement", "parallel")
class ParallelBlock:
    slots = {"norm": "norm", "mixer": "mixer", "ffn": "ffn"}
    optional = ("ffn",)
    takes_pending = False

    def __init__(self, norm, mixer, ffn=None):
        self.norm, self.mixer, self.ffn = norm, mixer, ffn

    def run(self, residual, delta, step, cache, writes_cache):
        """The sum goes into the 32-bit residual here (a mixer that says ``adds_to_residual`` does it in
        its own last kernel), so there is nothing left for the next norm to add: returns None."""
        h = self.norm.add_norm(residual, delta, "norm.parallel")
        if getattr(self.mixer, "adds_to_residual", False):
            # (the mixer calls the feed-forward when it suits it: beside a member that runs on a stream of its own)
            ffn = (lambda: self.ffn.forward(h, step)) if self.ffn is not None else None
            self.mixer.forward(h, step, cache, writes_cache, add_to=(residual, ffn))
        else:
            f = self.ffn.forward(h, step) if self.ffn is not None else None
            m = self.mixer.forward(h, step, cache, writes_cache)
            native.pair_rmsnorm_add(residual[: m.shape[0]], m, None, None, None, f, 0.0)
        return None
