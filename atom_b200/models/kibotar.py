"""Kibotar: a decoder-only model whose layers are listed one by one in config.json and of which a span may run
several times in a row on the same tensors.  The embedding adds a row chosen by the pair (previous token, token).
Every layer has a norm before AND after each sub-block, and its mixer reads every token blended with the token before
it (a token shift).  The mixer is gated linear attention, attention through a cached latent without positions (with a
gate number per head), or grouped-query attention over a sliding window and pooled blocks before it (rotary positions
stretched by wavelength, a sink of score zero, weights mixed over the heads, an output gate, biases); the feed-forward
is dense with relu squared, or absent.

config.json:  ``architecture`` "Kibotar"; ``vocab``, ``width``; ``norm.eps``;
``embedding``: scale, bigram {buckets, mul_prev, mul_cur}
``layers``: entries with ``type`` ("gla" | "latent_attention" | "attention"), ``mixer``, ``mlp`` (or null)
  gla mixer:               heads, dim, vdim, tau                       (the decay's rank from the tensor a1's shape)
  latent_attention mixer:  heads, dim, vdim, kv_rank, scale
  attention mixer:         heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, low, high, original}}
                           (absent: no rotation; scaling absent: plain frequencies), mask {size, pool} (absent: every
                           earlier token is seen; pool absent or 0: nothing is pooled)
  mlp: {kind "dense", ff}
``loop`` {start, stop, times} (absent: every layer runs once): layers start .. stop-1 run ``times`` times in a row, every
  pass on a cache of its own; row t of ``loop.step`` is added to the stream right before pass t's first layer.

Tensors: ``embed`` (also the output matrix), ``bigram`` [buckets + 1, width], ``loop.step`` [times, width],
``final.norm``, per layer ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``, ``l<i>.shift`` and
  gla:               ``l<i>.mix.{q,k,v,g,o,norm,a1,a2,a2.b}``
  latent_attention:  ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}``
  attention:         ``l<i>.mix.{q,k,v,o}`` with ``.b`` each, ``l<i>.mix.{talk,g}``
  dense:             ``l<i>.mlp.{up,down}``
Matrices are [out, in].

  x = embed[token] * scale + bigram[(previous * mul_prev + token * mul_cur) mod buckets]     (row ``buckets`` first)
  per layer run:  h = shift(rmsnorm(x; norm1));  x += rmsnorm(mixer(h); norm1b);
                  x += rmsnorm(mlp(rmsnorm(x; norm2)); norm2b)                               (if it has one)
  logits = embed rmsnorm(x; final.norm)
The mixers' formulas stand in parts/gla.py, parts/latent_attention.py and parts/pooled_attention.py, the shift's in
parts/token_shifted.py, the embedding's in parts/embedding.py (pair_embedding).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig, cfg_get, cfg_positive
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..parts.token_shifted import token_shifted_spec
from .registry import register_architecture

# Nothing in the design bounds a position (angles are computed from the position itself); a request's length is
# bounded by the engine's max_model_len, which defaults to this many tokens.
_DEFAULT_MAX_LEN = 32768
_MAX_POSITION = 1 << 24        # positions are exact in 32-bit floats up to here


@dataclass(frozen=True)
class GlaMixer:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: Optional[float]
    rot_dims: int
    rot_scaling: Optional[Tuple[float, float, float, float]]     # factor, low, high, original
    window: Optional[int]
    pool: Optional[int]


@dataclass(frozen=True)
class KibotarLayer:
    type: str
    mixer: Any                       # GlaMixer | LatentMixer | AttentionMixer
    ff: Optional[int]                # dense feed-forward's inner size (None: no feed-forward)


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


def _gla(m: Mapping, w: str, rank: Optional[int]) -> GlaMixer:
    if rank is None:
        rank = _count(m, "rank", w)          # (without a checkpoint the decay's rank is a key)
    tau = _number(m, "tau", w)
    if tau <= 0:
        raise ConfigError(f"config.json: {w}tau must be positive, got {tau}")
    return GlaMixer(heads=_count(m, "heads", w), dim=_count(m, "dim", w), vdim=_count(m, "vdim", w), tau=tau, rank=rank)


def _latent(m: Mapping, w: str) -> LatentMixer:
    return LatentMixer(heads=_count(m, "heads", w), dim=_count(m, "dim", w), vdim=_count(m, "vdim", w),
                       kv_rank=_count(m, "kv_rank", w), scale=_number(m, "scale", w))


def _attention(m: Mapping, w: str) -> AttentionMixer:
    base, dims, scaling = None, 0, None
    if m.get("rot") is not None:
        rot = _obj(m, "rot", w)
        base, dims = _number(rot, "base", w + "rot."), _count(rot, "dims", w + "rot.", 0)
        if base <= 1.0:
            raise ConfigError(f"config.json: {w}rot.base must exceed 1, got {base}")
        if rot.get("scaling") is not None:
            sc = _obj(rot, "scaling", w + "rot.")
            scaling = tuple(_number(sc, k, w + "rot.scaling.") for k in ("factor", "low", "high", "original"))
            if scaling[0] <= 0 or scaling[1] == scaling[2] or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
                raise ConfigError(f"config.json: {w}rot.scaling needs positive numbers and low != high")
    window, pool = None, None
    if m.get("mask") is not None:
        mask = _obj(m, "mask", w)
        window = _count(mask, "size", w + "mask.")
        if mask.get("pool") is not None:
            pool = _count(mask, "pool", w + "mask.", 0) or None
    out = AttentionMixer(heads=_count(m, "heads", w), kv_heads=_count(m, "kv_heads", w), dim=_count(m, "dim", w),
                         vdim=_count(m, "vdim", w), scale=_number(m, "scale", w), rot_base=base, rot_dims=dims,
                         rot_scaling=scaling, window=window, pool=pool)
    if out.heads % out.kv_heads:
        raise ConfigError(f"config.json: {w}heads ({out.heads}) must be a multiple of kv_heads ({out.kv_heads})")
    if out.rot_dims % 2 or out.rot_dims > out.dim:
        raise ConfigError(f"config.json: {w}rot.dims ({out.rot_dims}) must be even and at most dim ({out.dim})")
    return out


@dataclass(frozen=True)
class KibotarConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    embed_scale: float = 1.0
    buckets: int = 1
    mul_prev: int = 0
    mul_cur: int = 0
    layers: Tuple[KibotarLayer, ...] = ()
    loop: Optional[Tuple[int, int, int]] = None        # start, stop, times

    ARCHITECTURE: ClassVar[str] = "Kibotar"

    @classmethod
    def from_dict(cls, d: Dict[str, Any], shapes: Optional[Mapping[str, Tuple[int, ...]]] = None) -> "KibotarConfig":
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
            if kind == "gla":
                rank = None
                if shapes is not None:
                    a1 = shapes.get(f"l{i}.mix.a1")
                    if a1 is None or len(a1) != 2:
                        raise ConfigError(f"checkpoint: tensor l{i}.mix.a1 [rank, width] gives the decay's rank and is missing")
                    rank = int(a1[0])
                mixer = _gla(m, w + "mixer.", rank)
            elif kind == "latent_attention":
                mixer = _latent(m, w + "mixer.")
            elif kind == "attention":
                mixer = _attention(m, w + "mixer.")
            else:
                raise ConfigError(f"config.json: {w}type {kind!r} is not supported (gla, latent_attention, attention)")
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {w}mlp must be null or an object of kind 'dense'")
                ff = _count(mlp, "ff", w + "mlp.")
            layers.append(KibotarLayer(kind, mixer, ff))
        loop = None
        if d.get("loop") is not None:
            lp = _obj(d, "loop", "")
            loop = (_count(lp, "start", "loop.", 0), _count(lp, "stop", "loop.", 0), _count(lp, "times", "loop."))
            if not loop[0] <= loop[1] <= len(layers):
                raise ConfigError(f"config.json: loop runs layers {loop[0]} .. {loop[1]} - 1 of {len(layers)}")
            if loop[0] == loop[1]:
                loop = None                  # (an empty span: nothing runs twice and nothing is added)
        eps = _number(_obj(d, "norm", ""), "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        emb = _obj(d, "embedding", "")
        big = _obj(emb, "bigram", "embedding.")
        return cls(architecture=cls.ARCHITECTURE, vocab=cfg_positive("vocab", cfg_get(d, "vocab", int)),
                   width=cfg_positive("width", cfg_get(d, "width", int)), norm_eps=eps,
                   embed_scale=_number(emb, "scale", "embedding.") if emb.get("scale") is not None else 1.0,
                   buckets=_count(big, "buckets", "embedding.bigram."),
                   mul_prev=_count(big, "mul_prev", "embedding.bigram.", 0),
                   mul_cur=_count(big, "mul_cur", "embedding.bigram.", 0), layers=tuple(layers), loop=loop)

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps},
                               "embedding": {"scale": self.embed_scale,
                                             "bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev,
                                                        "mul_cur": self.mul_cur}},
                               "layers": []}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        for L in self.layers:
            m = L.mixer
            if L.type == "gla":
                mixer: Dict[str, Any] = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "tau": m.tau, "rank": m.rank}
            elif L.type == "latent_attention":
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.rot_base is not None:
                    mixer["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
                    if m.rot_scaling is not None:
                        mixer["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), m.rot_scaling))
                if m.window is not None:
                    mixer["mask"] = {"size": m.window}
                    if m.pool is not None:
                        mixer["mask"]["pool"] = m.pool
            out["layers"].append({"type": L.type, "mixer": mixer,
                                  "mlp": None if L.ff is None else {"kind": "dense", "ff": L.ff}})
        return out

    def run_order(self):
        """(layer, cache slot, number of the pass if the entry begins one) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, i, None) for i in range(n)]
        start, stop, times = self.loop
        out = [(i, i, None) for i in range(start)]
        slot = start
        for t in range(times):
            for i in range(start, stop):
                out.append((i, slot, t if i == start else None))
                slot += 1
        for i in range(stop, n):
            out.append((i, slot, None))
            slot += 1
        return out


def build_kibotar_spec(cfg: KibotarConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": (name,)})
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}"
        m = L.mixer
        if L.type == "gla":
            mixer = PartSpec(
                "gated_linear_attention",
                {"hidden_size": W, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "decay_rank": m.rank,
                 "tau": m.tau, "norm_eps": eps},
                {"in.weight": tuple(f"{p}.mix.{n}" for n in ("q", "k", "v", "g", "a1")), "a2.weight": (f"{p}.mix.a2",),
                 "a2.bias": (f"{p}.mix.a2.b",), "norm": (f"{p}.mix.norm",), "o.weight": (f"{p}.mix.o",)})
        elif L.type == "latent_attention":
            mixer = PartSpec(
                "latent_attention",
                {"hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": 0, "value_dim": m.vdim,
                 "q_rank": None, "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": eps, "position": None,
                 "gate": "head"},
                {"in.weight": tuple(f"{p}.mix.{n}" for n in ("q", "dkv", "g")), "dkv.norm": (f"{p}.mix.dkv.norm",),
                 "uk.weight": (f"{p}.mix.uk",), "uv.weight": (f"{p}.mix.uv",), "o.weight": (f"{p}.mix.o",)})
        else:
            position = None
            if m.rot_base is not None and m.rot_dims:
                scaling = None if m.rot_scaling is None else dict(zip(("factor", "low", "high", "original"), m.rot_scaling))
                position = PartSpec("rope_wavelength", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "scaling": scaling})
            mixer = PartSpec(
                "pooled_window_attention",
                {"hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim,
                 "value_dim": m.vdim, "scale": m.scale, "position": position, "window": m.window, "pool": m.pool,
                 "zero_sink": True, "talk": True, "gate": True, "bias": True},
                {"in.weight": tuple(f"{p}.mix.{n}" for n in ("q", "k", "v", "g")),
                 "qkv.bias": tuple(f"{p}.mix.{n}.b" for n in ("q", "k", "v")), "o.weight": (f"{p}.mix.o",),
                 "o.bias": (f"{p}.mix.o.b",), "talk": (f"{p}.mix.talk",)})
        parts = {"mixer_norm": norm(f"{p}.norm1"), "mixer": token_shifted_spec(W, mixer, f"{p}.shift"),
                 "mixer_post_norm": norm(f"{p}.norm1b")}
        if L.ff is not None:
            parts["ffn_norm"] = norm(f"{p}.norm2")
            parts["ffn"] = PartSpec("dense_relu2", {"hidden_size": W, "intermediate_size": L.ff},
                                    {"up.weight": (f"{p}.mlp.up",), "down.weight": (f"{p}.mlp.down",)})
            parts["ffn_post_norm"] = norm(f"{p}.norm2b")
        layers.append(LayerSpec("sandwich", parts))
    steps = None
    if cfg.loop is not None:
        steps = PartSpec("step_vectors", {"count": cfg.loop[2], "hidden_size": W}, {"table": ("loop.step",)})
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        max_position=_MAX_POSITION,
        default_max_len=_DEFAULT_MAX_LEN,
        embedding=PartSpec("pair_embedding",
                           {"vocab_size": cfg.vocab, "hidden_size": W, "buckets": cfg.buckets, "mul_prev": cfg.mul_prev,
                            "mul_cur": cfg.mul_cur, "scale": cfg.embed_scale},
                           {"weight": ("embed",), "pairs": ("bigram",)}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(layer=i, cache=slot, add_step=t) for i, slot, t in cfg.run_order()),
        final_norm=norm("final.norm"),
        lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": True}),
        stream_steps=steps,
        # (a span that is empty runs nothing twice; its vectors, if the checkpoint holds any, are not read)
        ignored_tensors=() if steps is not None else (r"^loop\.step$",),
    )


register_architecture(KibotarConfig.ARCHITECTURE, KibotarConfig.from_dict, build_kibotar_spec, reads_shapes=True)
