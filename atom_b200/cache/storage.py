"""Device arrays behind the cache manager's accounting.

For every page group one array per entry that its mixers declare (CacheNeed.entries):
[slots, pages, *shape with the page's tokens before the last axis], e.g. keys and values of
(kv heads, head size) each as [slots, pages, kv heads, page size, head size].  And one array
[state slots, *shape] per cache slot whose mixer keeps fixed-size state, zero when a request is
admitted.  ``view(slot)`` is what a mixer gets for its run entry."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from .manager import CacheManager


@dataclass
class CacheView:
    slot: int
    group: int = -1                       # page group (index into StepContext.block_tables)
    page_size: int = 0
    pages: Dict[str, torch.Tensor] = field(default_factory=dict)   # entry name -> [pages, ..., page size, last]
    state: Optional[torch.Tensor] = None     # [state slots, *shape]: the array of a need of kind "state" with a shape
    states: Dict[str, torch.Tensor] = field(default_factory=dict)  # named state arrays, each [state slots, *shape]
    # rows kept per whole block of positions (CacheNeed.block_entries): their page group and arrays, a row where a
    # token group has a token
    block_group: int = -1
    block_pages: Dict[str, torch.Tensor] = field(default_factory=dict)

    def member(self, name: str) -> "CacheView":
        """The view of one member of a mixer whose need was put together with ``CacheNeed.merged``: the pages,
        and the state arrays ``<name>.<array>`` under their own names (``<name>.state`` as ``state``)."""
        own = {k[len(name) + 1:]: v for k, v in self.states.items() if k.startswith(name + ".")}
        return CacheView(self.slot, self.group, self.page_size, self.pages, own.pop("state", None), own,
                         self.block_group, self.block_pages)

    @property
    def k_pages(self) -> Optional[torch.Tensor]:   # [pages, kv heads, page size, head size]
        return self.pages.get("k")

    @property
    def v_pages(self) -> Optional[torch.Tensor]:
        return self.pages.get("v")


def _entry_dtype(entry, compute: torch.dtype) -> torch.dtype:
    return compute if entry.dtype == "compute" else getattr(torch, entry.dtype)


def _page_shape(entry, page_size: int):
    return tuple(entry.shape[:-1]) + (page_size, entry.shape[-1])


class CacheStorage:
    def __init__(self, manager: CacheManager, dtype: torch.dtype, device):
        self.manager = manager
        self.arrays = []
        self._views: Dict[int, CacheView] = {}
        self._states = []
        ps = manager.page_size
        for g in manager.groups:
            per_entry = {}
            for e in g.entries:
                a = torch.zeros((len(g.slots), g.pool.num_pages) + _page_shape(e, ps),
                                dtype=_entry_dtype(e, dtype), device=device)
                self.arrays.append(a)
                per_entry[e.name] = a
            for i, slot in enumerate(g.slots):
                if g.block:        # (the slot's token group stands before it in the list: its view exists)
                    self._views[slot].block_group = g.index
                    self._views[slot].block_pages = {n: a[i] for n, a in per_entry.items()}
                else:
                    self._views[slot] = CacheView(slot, g.index, ps, {n: a[i] for n, a in per_entry.items()})
        n_slots = manager.state_slots.num_slots
        for slot, need in manager.state_needs.items():
            view = self._views.get(slot)
            if view is None:
                view = self._views[slot] = CacheView(slot)
            if need.kind == "state" and need.state_shape:
                sdt = dtype if need.state_dtype == "compute" else getattr(torch, need.state_dtype)
                view.state = torch.zeros((n_slots,) + tuple(need.state_shape), dtype=sdt, device=device)
                self.arrays.append(view.state)
                self._states.append(view.state)
            for e in need.states:
                st = torch.zeros((n_slots,) + tuple(e.shape), dtype=_entry_dtype(e, dtype), device=device)
                view.states[e.name] = st
                self.arrays.append(st)
                self._states.append(st)
        if self._states:
            manager.admit_hooks.append(self.clear_state)

    def clear_state(self, state_slot: int) -> None:
        """Zeroes a request slot's rows in every state array.  Runs when a request is admitted (a
        preempted request that comes back included), so a mixer finds zeros at a request's first
        token whoever held the slot before."""
        for st in self._states:
            st[state_slot].zero_()

    def view(self, slot: int) -> Optional[CacheView]:
        return self._views.get(slot)

    def get(self, slot: int) -> Optional[CacheView]:   # mapping-style access used by Model.forward
        return self._views.get(slot)

    def bytes(self) -> int:
        return sum(a.numel() * a.element_size() for a in self.arrays)

    @staticmethod
    def bytes_per_page(manager: CacheManager, dtype: torch.dtype) -> int:
        """Bytes that one more page in every group costs."""
        total = 0
        for g in manager.groups:
            for e in g.entries:
                n = manager.page_size
                for d in e.shape:
                    n *= d
                b = len(g.slots) * n * torch.empty((), dtype=_entry_dtype(e, dtype)).element_size()
                total += -(-b // g.block) if g.block else b
        return total
