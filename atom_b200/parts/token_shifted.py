"""A mixer behind a token shift: what the member mixer reads is every token blended with the token before it in its
request,
   h_t <- h_t + (h_(t-1) - h_t) * mu        element by element, h_(t-1) as it was before the blend, zeros before the
                                            request's first token,
for any registered mixer kind.  The last h of a step is part of the request's state (one row of the activation type in
its state slot, beside whatever the member keeps); the member's parameters appear under ``mixer.``, the blend vector as
``mu``.  The blend is formed in 32-bit and rounded once.
"""
from __future__ import annotations

from typing import Dict

from .. import native
from . import registry
from .base import Mixer
from .registry import register
from .spec import CacheEntry, CacheNeed, ParamSpec, PartSpec

_MEMBER = "mixer"


def token_shifted_spec(hidden_size: int, member: PartSpec, mu_source: str) -> PartSpec:
    """The PartSpec of ``member`` behind a token shift: its checkpoint names move under ``mixer.``."""
    sources = {f"{_MEMBER}.{k}": v for k, v in member.sources.items()}
    sources["mu"] = (mu_source,)
    return PartSpec("token_shifted", {"hidden_size": hidden_size, "member": PartSpec(member.kind, dict(member.args))},
                    sources)


@register("mixer", "token_shifted")
class TokenShifted(Mixer):
    def __init__(self, hidden_size: int, member: PartSpec):
        self.hidden_size = hidden_size
        self.member = registry.build("mixer", member)
        self.defers_output = bool(getattr(self.member, "defers_output", False))

    @property
    def graph_safe(self) -> bool:
        return self.member.graph_safe

    def params(self) -> Dict[str, ParamSpec]:
        p = {f"{_MEMBER}.{k}": v for k, v in self.member.params().items()}
        p["mu"] = ParamSpec((1, self.hidden_size), role="vector", init="half", rows=(1,), members_lack_axis=True)
        return p

    def cache_need(self) -> CacheNeed:
        own = CacheNeed("state", states=(CacheEntry("last", (self.hidden_size,), "compute"),))
        return CacheNeed.merged({"shift": own, _MEMBER: self.member.cache_need()})

    def bind(self, tensors, rt):
        self.rt = rt
        self.w_mu = tensors["mu"]
        n = len(_MEMBER) + 1
        self.member.bind({k[n:]: v for k, v in tensors.items() if k.startswith(_MEMBER + ".")}, rt)

    def after_load(self) -> None:
        self.member.after_load()

    def launch_plan(self, step) -> None:
        self.member.launch_plan(step)

    def forward(self, x, step, cache, writes_cache, **kw):
        T, W = x.shape
        mixed = self.rt.workspace.get("shift.mixed", (1, T, W), self.rt.dtype)
        native.token_shift_mix(mixed, x, self.w_mu, cache.states["shift.last"], step.seq_of_token, step.cu_q,
                               step.state_slots, writes_cache)
        return self.member.forward(mixed[0], step, cache.member(_MEMBER), writes_cache, **kw)
