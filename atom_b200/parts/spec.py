"""Data that describes a model: parts, their parameters, the layers and their run order.

An architecture (``atom_b200/models/<name>.py``) turns its typed configuration into a
``ModelSpec``.  The spec is plain data: which mixer, feed-forward, norm and position
encoding each layer has, with the sizes and constants each takes as arguments, from which
checkpoint tensors each parameter is read, and the order in which layers run.  Nothing in
the engine, the cache manager or the loader knows an architecture by name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class ParamSpec:
    """One parameter tensor of a part.

    role   "matrix": operand of a matrix product, held in the engine's compute type.
           "vector": norm weight or bias; held in bfloat16 unless stored (or run) in 32-bit.
           "table":  integer table, held as int32.
    init   distribution of the random-weights mode: "normal" N(0, 0.02^2), "norm" U(0.8, 1.2),
           "zeros", "half" U(0.25, 0.75), "eye" (identity plus N(0, 0.02^2), square matrices).
    rows   when the parameter is several checkpoint tensors stacked along one axis, their extents
           along it.
    stack_dim   that axis (0: rows under one another, as q/k/v; 1: side by side).
    members_lack_axis   the stacked checkpoint tensors have no such axis of their own (each is one
           slice: vectors [n] stacked into [m, n]); every extent in ``rows`` is then 1.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    rows: Optional[Tuple[int, ...]] = None
    stack_dim: int = 0
    members_lack_axis: bool = False


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by registry key with its constructor arguments.

    sources maps a parameter name of the part to the checkpoint tensor names it is read
    from (more than one: stacked along the parameter's ``stack_dim`` in that order).  A parameter absent from
    ``sources`` is not read from the checkpoint (e.g. a tied output matrix).
    """

    kind: str
    args: Dict[str, Any] = field(default_factory=dict)
    sources: Dict[str, Tuple[str, ...]] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement and the parts it is put together from, by the names under which the
    arrangement knows them.  Which names there are, and of which category each is, is the
    arrangement's affair (its ``slots``): "prenorm" has mixer_norm, mixer, ffn_norm and ffn; another
    arrangement may have four norms, no feed-forward, or two mixers."""

    arrangement: str
    parts: Mapping[str, PartSpec]
    # constants of the arrangement itself (keyword arguments of its constructor beside the parts)
    args: Mapping[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.arrangement, tuple(sorted(self.parts))))


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order: run layer ``layer`` on cache ``cache``.

    A layer may be named by several entries (its weights are shared); ``cache`` names the
    cache slot the mixer uses, and with ``writes_cache=False`` the mixer only reads what
    another entry wrote to that slot in the same step.
    """

    layer: int
    cache: int
    writes_cache: bool = True
    # Row of the model's ``stream_steps`` table that is added to the residual stream right before this entry runs
    # (None: nothing is added): a design that runs a span of layers several times marks every pass this way.
    add_step: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    # Regular expressions of checkpoint tensor names that are neither read nor reported.
    ignored_tensors: Tuple[str, ...] = ()
    # (name, other): a checkpoint tensor that the model does not read but that may be present when it
    # is, element for element, the tensor ``other``; present and different is a loading error.
    duplicate_tensors: Tuple[Tuple[str, str], ...] = ()
    eos_token_ids: Tuple[int, ...] = ()
    # Longest request the engine takes when its own max_model_len is not given; None: max_position
    # (for models whose design names no longest sequence, max_position is the engine's own bound).
    default_max_len: Optional[int] = None
    # A part of category "stream" that holds vectors of the residual's width which run entries add to the stream
    # (``RunEntry.add_step``); None: the design has none.
    stream_steps: Optional[PartSpec] = None


@dataclass(frozen=True)
class CacheEntry:
    """One array that a mixer keeps in pages: ``shape`` per token, in the compute type unless
    ``dtype`` names a torch type.  In the page array the token axis stands before the last axis:
    (kv heads, head size) is stored as [pages, kv heads, page size, head size], a single row (r,)
    as [pages, page size, r]."""

    name: str
    shape: Tuple[int, ...]
    dtype: str = "compute"


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per request between steps.

    kind "pages": ``entries`` for every position (or for the last ``window`` positions, and with
                  ``keep_first`` also for the request's first positions, which a window never drops),
                  held in pages.  Giving ``num_kv_heads`` and ``head_dim`` instead stands for the two
                  entries "k" and "v" of that shape each.
    kind "state": one array of fixed shape per request, held in a slot.
    A need of pages may also keep ``block_entries``: one row of these arrays for every whole block of ``block``
    consecutive positions (block b holds positions b * block .. b * block + block - 1; a request of n positions has
    n // block rows), in pages of a group of their own that a window never gives back.
    Either kind may also name ``states``: arrays of fixed shape per request (``CacheEntry`` with the
    whole shape, in the compute type unless ``dtype`` says otherwise), held in the request's slot and
    all zeros at the request's first token.  A mixer that keeps pages and a recurrent state side by
    side declares kind "pages" with ``states``; ``merged`` puts two mixers' needs together.
    """

    kind: str
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    keep_first: int = 0
    state_shape: Tuple[int, ...] = ()
    state_dtype: str = "float32"
    entries: Tuple[CacheEntry, ...] = ()
    states: Tuple[CacheEntry, ...] = ()
    block: int = 0
    block_entries: Tuple[CacheEntry, ...] = ()

    def __post_init__(self):
        if bool(self.block_entries) != (self.block > 0) or (self.block_entries and self.kind != "pages"):
            raise ValueError("rows per block need a block length and a need of pages")
        names = [e.name for e in self.states]
        if len(set(names)) != len(names) or any(not e.shape for e in self.states):
            raise ValueError(f"state arrays need distinct names and a shape: {self.states}")
        if self.kind == "pages" and not self.entries:
            if self.num_kv_heads <= 0 or self.head_dim <= 0:
                raise ValueError("a 'pages' cache need names its entries, or kv heads and head size")
            shape = (self.num_kv_heads, self.head_dim)
            object.__setattr__(self, "entries", (CacheEntry("k", shape), CacheEntry("v", shape)))
        if self.kind == "pages":
            names = [e.name for e in self.entries]
            if len(set(names)) != len(names) or any(not e.shape for e in self.entries):
                raise ValueError(f"cache entries need distinct names and a shape per token: {self.entries}")

    def block_group_key(self) -> Optional[Tuple]:
        return ("blocks", self.block_entries, self.block) if self.block_entries else None

    def group_key(self) -> Tuple:
        if self.kind == "pages":
            return ("pages", self.entries, self.window) + ((self.keep_first,) if self.window and self.keep_first else ())
        return ("state", self.state_shape, self.state_dtype)

    @property
    def keeps_state(self) -> bool:
        return self.kind == "state" or bool(self.states)

    @staticmethod
    def merged(needs: Mapping[str, Optional["CacheNeed"]]) -> Optional["CacheNeed"]:
        """The one need of a mixer made of several (name -> need of each): the pages of the one member
        that keeps pages (more than one is refused: they would have to share a block table and a
        window) and every member's state arrays, named ``<member>.<array>``; a member of kind "state"
        gives the array ``<member>.state``."""
        pages = [(n, c) for n, c in needs.items() if c is not None and c.kind == "pages"]
        if len(pages) > 1:
            raise ValueError(f"more than one member keeps pages: {[n for n, _ in pages]}")
        states = []
        for n, c in needs.items():
            if c is None:
                continue
            if c.kind == "state" and c.state_shape:
                states.append(CacheEntry(f"{n}.state", tuple(c.state_shape), c.state_dtype))
            states += [CacheEntry(f"{n}.{e.name}", e.shape, e.dtype) for e in c.states]
        if pages:
            c = pages[0][1]
            return CacheNeed("pages", window=c.window, keep_first=c.keep_first, entries=c.entries, states=tuple(states),
                             block=c.block, block_entries=c.block_entries)
        if states:
            return CacheNeed("state", states=tuple(states))
        return None
