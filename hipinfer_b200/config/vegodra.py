"""`VegodraConfig`: the config.json of the Vegodra decoder, typed and checked.

A Vegodra model is a list of layers, each a parallel block (one norm, read by a sequence mixer and a feed-forward):

    architecture    "Vegodra"
    vocab, width
    norm.eps                        of every norm of the model
    max_positions                   optional: the longest sequence (absent: DEFAULT_MAX_POSITIONS)
    layers[i].type                  "latent_attention", "attention" or "gla"
    layers[i].mixer                 latent_attention: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {base, dims}
                                    attention: heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size} (chunks of
                                    that many positions; absent: every earlier token is seen), kv_from (index of the
                                    layer whose keys and values this one reads; absent: its own)
                                    gla: heads, dim, vdim, tau
    layers[i].mlp                   null, or {kind: "dense", ff}

What config.json does not hold is read from a tensor's shape (the rank of the decay's low-rank pair of a gla mixer).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take

DEFAULT_MAX_POSITIONS = 131072


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int

    def to_dict(self):
        return dict(base=self.base, dims=self.dims)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: RotaryConfig

    def to_dict(self):
        return dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, q_rank=self.q_rank,
                    kv_rank=self.kv_rank, scale=self.scale, rot=self.rot.to_dict())


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotaryConfig
    chunk: Optional[int] = None       # mask.size; None: no mask beyond the causal one
    kv_from: Optional[int] = None

    def to_dict(self):
        d = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale, rot=self.rot.to_dict())
        if self.chunk is not None:
            d["mask"] = dict(size=self.chunk)
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class GlaConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: Optional[int] = None  # used by the random-weights mode; a checkpoint's tensor shapes decide otherwise

    def to_dict(self):
        d = dict(heads=self.heads, dim=self.dim, vdim=self.vdim, tau=self.tau)
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        return d


@dataclass(frozen=True)
class VegodraLayerConfig:
    type: str                         # "latent_attention" | "attention" | "gla"
    mixer: Any
    ff: Optional[int] = None          # width of the dense feed-forward; None: the layer has none

    def to_dict(self):
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=None if self.ff is None else dict(kind="dense", ff=self.ff))


def _sub(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _rot(m, where, limit, what):
    r = _sub(m, "rot", where + "mixer.")
    rot = RotaryConfig(take(r, "base", float, positive=True), take(r, "dims", int))
    if rot.dims < 0 or rot.dims % 2 or rot.dims > limit:
        raise ConfigError(f"config.json: {where}mixer.rot.dims = {rot.dims} must be even and at most {what} = {limit}")
    return rot


@dataclass(frozen=True)
class VegodraConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[VegodraLayerConfig, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VegodraConfig":
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: key 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = take(L, "type", str)
            m = _sub(L, "mixer", where)
            pos = lambda key: take(m, key, int, positive=True)
            if kind == "latent_attention":
                rot_dim = pos("rot_dim")
                mixer = LatentAttentionConfig(pos("heads"), pos("dim"), rot_dim, pos("vdim"), pos("q_rank"), pos("kv_rank"),
                                              take(m, "scale", float, positive=True), _rot(m, where, rot_dim, "rot_dim"))
            elif kind == "attention":
                heads, kv, dim = pos("heads"), pos("kv_heads"), pos("dim")
                if heads % kv:
                    raise ConfigError(f"config.json: {where}mixer: {heads} heads are not a multiple of {kv} kv_heads")
                mask = m.get("mask")
                if mask is not None and not isinstance(mask, dict):
                    raise ConfigError(f"config.json: {where}mixer.mask must be an object or null")
                chunk = take(mask, "size", int, None, positive=True) if mask else None
                src = take(m, "kv_from", int, None)
                if src is not None:
                    if not (0 <= src < i) or raw[src].get("type") != "attention" or raw[src].get("mixer", {}).get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}mixer.kv_from = {src} must name an earlier attention layer "
                                          f"with keys and values of its own")
                mixer = ChunkedAttentionConfig(heads, kv, dim, pos("vdim"), take(m, "scale", float, positive=True),
                                               _rot(m, where, dim, "dim"), chunk, src)
            elif kind == "gla":
                mixer = GlaConfig(pos("heads"), pos("dim"), pos("vdim"), take(m, "tau", float, positive=True),
                                  take(m, "decay_rank", int, None, positive=True))
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not known (known: 'latent_attention', 'attention', 'gla')")
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}mlp must be an object or null")
                if take(mlp, "kind", str) != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp['kind']!r} is not known (known: 'dense')")
                ff = take(mlp, "ff", int, positive=True)
            layers.append(VegodraLayerConfig(kind, mixer, ff))
        for i, L in enumerate(layers):
            if L.type == "attention" and L.mixer.kv_from is not None:
                s, m = layers[L.mixer.kv_from].mixer, L.mixer
                if (s.kv_heads, s.dim, s.vdim, s.rot) != (m.kv_heads, m.dim, m.vdim, m.rot):
                    raise ConfigError(f"config.json: layers[{i}] reads the keys and values of layers[{m.kv_from}], whose "
                                      f"kv_heads, dim, vdim or rotation differ")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos)
        return cls(architecture=d["architectures"][0] if "architectures" in d else d["architecture"],
                   vocab=take(d, "vocab", int, positive=True), width=take(d, "width", int, positive=True),
                   norm_eps=take(_sub(d, "norm", ""), "eps", float, positive=True), layers=tuple(layers),
                   max_positions=take(d, "max_positions", int, DEFAULT_MAX_POSITIONS, positive=True), eos_token_ids=eos_ids)

    def to_dict(self) -> Dict[str, Any]:
        d = dict(architecture=self.architecture, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps),
                 layers=[L.to_dict() for L in self.layers])
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
