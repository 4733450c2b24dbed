"""Simivik: a decoder-only model whose layers are listed one by one in config.json.  Every layer is pre-norm with
norm weights stored around zero (the factor is 1 + w); its mixer is either grouped-query attention behind a short
causal convolution on q, k and v (partial rotation, capped scores, a sliding window that always keeps a request's
first tokens) or lightning attention (a decayed matrix state per head, gated output); its feed-forward is dense
with relu squared, a mixture of gated experts, or absent.  A layer may run another layer's tensors on a cache of
its own.

config.json:  ``architecture`` "Simivik"; ``vocab``, ``width``; ``norm.eps``;
``layers``: entries with ``type`` ("attention" | "lightning"), ``mixer``, ``mlp`` (or null), optional ``weights_of``.
  attention mixer: heads, kv_heads, dim, vdim, scale, softcap (absent or 0: none), conv (taps; absent or 0: none),
      rot {base, dims} (absent: no rotation), mask {size, keep_first} (absent: every earlier token is seen)
  lightning mixer: heads, dim, vdim, decay (one number per head; a single number stands for all heads)
  mlp: {kind "dense", ff}  |  {kind "moe", router {experts, top}, expert {ff}, shared {ff} (absent: none)}

Tensors: ``embed`` (also the output matrix), ``final.norm``, per layer ``l<i>.norm1``, ``l<i>.norm2`` and
  attention: ``l<i>.mix.{q,k,v,o}``, with a convolution ``l<i>.mix.{q,k,v}.conv`` [channels, taps]
  lightning: ``l<i>.mix.{q,k,v,g,o,norm}``
  dense:     ``l<i>.mlp.{up,down}``
  moe:       ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.shared.{gate,up,down,sg}``
Matrices are [out, in].

  x = embed[token]
  per layer:  x += mixer(rmsnorm(x; 1 + norm1));   x += mlp(rmsnorm(x; 1 + norm2))   (if it has one)
  logits = embed rmsnorm(x; 1 + final.norm)
The mixers' formulas stand in parts/conv_attention.py and parts/lightning.py, the feed-forwards' in parts/mlp.py
(dense_relu2) and parts/moe.py (routed_experts).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig, cfg_get, cfg_positive
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import register_architecture

# Nothing in the design bounds a position (angles are computed from the position itself); a request's length is
# bounded by the engine's max_model_len, which defaults to this many tokens.
_DEFAULT_MAX_LEN = 32768
_MAX_POSITION = 1 << 24        # positions are exact in 32-bit floats up to here


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    taps: Optional[int]
    rot_base: Optional[float]
    rot_dims: int
    window: Optional[int]
    keep_first: int


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class Experts:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class SimivikLayer:
    type: str
    mixer: Any                       # AttentionMixer | LightningMixer
    ff: Optional[int]                # dense feed-forward's inner size
    moe: Optional[Experts]           # or a mixture of experts (both None: no feed-forward)
    weights_of: Optional[int] = None


def _obj(d: Mapping, key: str, where: str) -> Mapping:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


def _number(d: Mapping, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def _count(d: Mapping, key: str, where: str, least: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"config.json: {where}'{key}' must be an int >= {least}, got {v!r}")
    return v


def _attention(m: Mapping, w: str) -> AttentionMixer:
    rot = m.get("rot")
    base, dims = None, 0
    if rot is not None:
        rot = _obj(m, "rot", w)
        base, dims = _number(rot, "base", w + "rot."), _count(rot, "dims", w + "rot.", 0)
        if base <= 1.0:
            raise ConfigError(f"config.json: {w}rot.base must exceed 1, got {base}")
    window, keep = None, 0
    if m.get("mask") is not None:
        mask = _obj(m, "mask", w)
        window = _count(mask, "size", w + "mask.")
        keep = _count(mask, "keep_first", w + "mask.", 0) if mask.get("keep_first") is not None else 0
    cap = m.get("softcap")
    if cap is not None:
        cap = _number(m, "softcap", w)
        if cap < 0:
            raise ConfigError(f"config.json: {w}softcap must be positive, got {cap}")
        cap = cap or None                            # (0 stands for no cap, as an absent key does)
    taps = _count(m, "conv", w, 0) if m.get("conv") is not None else None
    taps = taps or None                              # (0 taps: no convolution)
    out = AttentionMixer(heads=_count(m, "heads", w), kv_heads=_count(m, "kv_heads", w), dim=_count(m, "dim", w),
                         vdim=_count(m, "vdim", w), scale=_number(m, "scale", w), softcap=cap, taps=taps,
                         rot_base=base, rot_dims=dims, window=window, keep_first=keep)
    if out.heads % out.kv_heads:
        raise ConfigError(f"config.json: {w}heads ({out.heads}) must be a multiple of kv_heads ({out.kv_heads})")
    if out.rot_dims % 2 or out.rot_dims > out.dim:
        raise ConfigError(f"config.json: {w}rot.dims ({out.rot_dims}) must be even and at most dim ({out.dim})")
    return out


def _lightning(m: Mapping, w: str) -> LightningMixer:
    heads = _count(m, "heads", w)
    decay = m.get("decay")
    if isinstance(decay, (int, float)) and not isinstance(decay, bool):
        decay = [decay] * heads                      # one number: the same decay for every head
    if not isinstance(decay, list) or len(decay) != heads or \
            any(isinstance(v, bool) or not isinstance(v, (int, float)) for v in decay):
        raise ConfigError(f"config.json: {w}decay must list one number per head ({heads})")
    return LightningMixer(heads=heads, dim=_count(m, "dim", w), vdim=_count(m, "vdim", w),
                          decay=tuple(float(v) for v in decay))


def _mlp(mlp, w: str):
    if mlp is None:
        return None, None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {w}mlp must be an object or null")
    kind = mlp.get("kind")
    if kind == "dense":
        return _count(mlp, "ff", w + "mlp."), None
    if kind == "moe":
        router = _obj(mlp, "router", w + "mlp.")
        e = Experts(experts=_count(router, "experts", w + "mlp.router."), top=_count(router, "top", w + "mlp.router."),
                    ff=_count(_obj(mlp, "expert", w + "mlp."), "ff", w + "mlp.expert."),
                    shared_ff=None if mlp.get("shared") is None
                    else _count(_obj(mlp, "shared", w + "mlp."), "ff", w + "mlp.shared."))
        if e.top > e.experts:
            raise ConfigError(f"config.json: {w}mlp.router.top ({e.top}) exceeds experts ({e.experts})")
        return None, e
    raise ConfigError(f"config.json: {w}mlp.kind {kind!r} is not supported (dense, moe)")


@dataclass(frozen=True)
class SimivikConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    layers: Tuple[SimivikLayer, ...] = ()

    ARCHITECTURE: ClassVar[str] = "Simivik"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SimivikConfig":
        entries = d.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            w = f"layers[{i}]."
            if not isinstance(e, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = e.get("type")
            m = _obj(e, "mixer", w)
            if kind == "attention":
                mixer = _attention(m, w + "mixer.")
            elif kind == "lightning":
                mixer = _lightning(m, w + "mixer.")
            else:
                raise ConfigError(f"config.json: {w}type {kind!r} is not supported (attention, lightning)")
            ff, moe = _mlp(e.get("mlp"), w)
            src = e.get("weights_of")
            if src is not None and (isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(entries)
                                    or src == i):
                raise ConfigError(f"config.json: {w}weights_of = {src!r} names no other layer")
            layers.append(SimivikLayer(kind, mixer, ff, moe, src))
        out_layers = tuple(layers)
        for i, L in enumerate(out_layers):
            j, seen = i, set()
            while out_layers[j].weights_of is not None:      # chains are followed; a loop is refused
                if j in seen:
                    raise ConfigError(f"config.json: layers[{i}].weights_of leads round in a circle")
                seen.add(j)
                j = out_layers[j].weights_of
            if j != i:
                o = out_layers[j]
                if (L.type, L.mixer, L.ff, L.moe) != (o.type, o.mixer, o.ff, o.moe):
                    raise ConfigError(f"config.json: layers[{i}] runs layer {j}'s tensors but has other sizes or constants")
        eps = _number(_obj(d, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        return cls(architecture=cls.ARCHITECTURE, vocab=cfg_positive("vocab", cfg_get(d, "vocab", int)),
                   width=cfg_positive("width", cfg_get(d, "width", int)), norm_eps=eps, layers=out_layers)

    def owner_of(self, i: int) -> int:
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
        return i

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "layers": []}
        for L in self.layers:
            m = L.mixer
            if L.type == "attention":
                mixer: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
                                         "scale": m.scale}
                if m.softcap is not None:
                    mixer["softcap"] = m.softcap
                if m.taps is not None:
                    mixer["conv"] = m.taps
                if m.rot_base is not None:
                    mixer["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
                if m.window is not None:
                    mixer["mask"] = {"size": m.window, "keep_first": m.keep_first}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            if L.moe is not None:
                mlp: Any = {"kind": "moe", "router": {"experts": L.moe.experts, "top": L.moe.top},
                            "expert": {"ff": L.moe.ff}}
                if L.moe.shared_ff is not None:
                    mlp["shared"] = {"ff": L.moe.shared_ff}
            else:
                mlp = None if L.ff is None else {"kind": "dense", "ff": L.ff}
            e = {"type": L.type, "mixer": mixer, "mlp": mlp}
            if L.weights_of is not None:
                e["weights_of"] = L.weights_of
            out["layers"].append(e)
        return out


def build_simivik_spec(cfg: SimivikConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", {"size": W, "eps": eps, "weight_offset": 1.0}, {"weight": (name,)})
    layers, index = [], {}
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            continue
        p = f"l{i}"
        m = L.mixer
        if L.type == "attention":
            position = None if m.rot_base is None or m.rot_dims == 0 else \
                PartSpec("rope_yarn", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "scaling": None})
            sources = {"qkv.weight": tuple(f"{p}.mix.{n}" for n in ("q", "k", "v")), "o.weight": (f"{p}.mix.o",)}
            if m.taps is not None:
                sources["conv.weight"] = tuple(f"{p}.mix.{n}.conv" for n in ("q", "k", "v"))
            mixer = PartSpec(
                "conv_window_attention",
                {"hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim,
                 "value_dim": m.vdim, "scale": m.scale, "softcap": m.softcap, "taps": m.taps, "position": position,
                 "window": m.window, "keep_first": m.keep_first},
                sources)
        else:
            mixer = PartSpec(
                "lightning_attention",
                {"hidden_size": W, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "decay": m.decay,
                 "norm_eps": eps},
                {"qkvg.weight": tuple(f"{p}.mix.{n}" for n in ("q", "k", "v", "g")), "norm": (f"{p}.mix.norm",),
                 "o.weight": (f"{p}.mix.o",)})
        parts = {"mixer_norm": norm(f"{p}.norm1"), "mixer": mixer}
        if L.ff is not None:
            parts["ffn_norm"] = norm(f"{p}.norm2")
            parts["ffn"] = PartSpec("dense_relu2", {"hidden_size": W, "intermediate_size": L.ff},
                                    {"up.weight": (f"{p}.mlp.up",), "down.weight": (f"{p}.mlp.down",)})
        elif L.moe is not None:
            e = L.moe
            sources = {"router.weight": (f"{p}.mlp.router",) + ((f"{p}.mlp.shared.sg",) if e.shared_ff else ()),
                       "gate_up.weight": tuple(f"{p}.mlp.e{j}.{n}" for j in range(e.experts) for n in ("gate", "up")),
                       "down.weight": tuple(f"{p}.mlp.e{j}.down" for j in range(e.experts))}
            if e.shared_ff:
                sources["shared.gate_up.weight"] = (f"{p}.mlp.shared.gate", f"{p}.mlp.shared.up")
                sources["shared.down.weight"] = (f"{p}.mlp.shared.down",)
            parts["ffn_norm"] = norm(f"{p}.norm2")
            parts["ffn"] = PartSpec(
                "routed_experts",
                {"hidden_size": W, "num_experts": e.experts, "top": e.top, "intermediate_size": e.ff,
                 "shared_size": e.shared_ff, "score": "sigmoid", "renormalize": False, "weight_on": "input",
                 "shared_gate": bool(e.shared_ff)},
                sources)
        index[i] = len(layers)
        layers.append(LayerSpec("prenorm_scaled", parts, {"residual_mult": 1.0}))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        max_position=_MAX_POSITION,
        default_max_len=_DEFAULT_MAX_LEN,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W}, {"weight": ("embed",)}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(layer=index[cfg.owner_of(i)], cache=i) for i in range(len(cfg.layers))),
        final_norm=norm("final.norm"),
        lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": True}),
    )


register_architecture(SimivikConfig.ARCHITECTURE, SimivikConfig.from_dict, build_simivik_spec)
