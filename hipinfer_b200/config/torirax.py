"""`ToriraxConfig`: the config.json of the Torirax decoder, typed and checked.

A Torirax model is a list of layers, each with one sequence mixer and, optionally, a feed-forward:

    architecture    "Torirax"
    vocab, width, max_positions
    embedding.scale                 the token embedding is multiplied by it
    norm.eps                        of every norm of the model
    layers[i].type                  "general_delta" (a delta-rule recurrence) or "attention" (differential attention)
    layers[i].mixer                 general_delta: heads, dim
                                    attention: heads, kv_heads, dim (query/key size of a map), vdim (value size), scale,
                                    diff (the constant of the differential combination), mask {size, keep_first} (a
                                    sliding window that keeps the first tokens; absent: every earlier token is seen),
                                    kv_from (index of the layer whose keys and values this one reads; absent: its own)
    layers[i].mlp                   null, or {kind: "dense", ff}

What config.json does not hold is read from a tensor's shape (the rank of the decay's low-rank pair): `decay_rank`
in a general_delta mixer is optional, used by the random-weights mode, and else left to the weights.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, take


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    dim: int
    decay_rank: Optional[int] = None

    def to_dict(self):
        d = dict(heads=self.heads, dim=self.dim)
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        return d


@dataclass(frozen=True)
class DiffAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: Optional[int] = None      # mask.size; None: no window
    keep_first: int = 0               # mask.keep_first
    kv_from: Optional[int] = None

    def to_dict(self):
        d = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale, diff=self.diff)
        if self.window is not None:
            d["mask"] = dict(size=self.window, keep_first=self.keep_first)
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class ToriraxLayerConfig:
    type: str                                   # "general_delta" | "attention"
    mixer: Any                                  # DeltaMixerConfig | DiffAttentionConfig
    ff: Optional[int] = None                    # width of the dense feed-forward; None: the layer has none

    def to_dict(self):
        return dict(type=self.type, mixer=self.mixer.to_dict(), mlp=None if self.ff is None else dict(kind="dense", ff=self.ff))


def _sub(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


@dataclass(frozen=True)
class ToriraxConfig(ModelConfig):
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[ToriraxLayerConfig, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ToriraxConfig":
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
            if kind == "general_delta":
                mixer = DeltaMixerConfig(take(m, "heads", int, positive=True), take(m, "dim", int, positive=True),
                                         take(m, "decay_rank", int, None, positive=True))
            elif kind == "attention":
                heads, kv = take(m, "heads", int, positive=True), take(m, "kv_heads", int, positive=True)
                if heads % kv:
                    raise ConfigError(f"config.json: {where}mixer: {heads} heads are not a multiple of {kv} kv_heads")
                mask = m.get("mask")
                if mask is not None and not isinstance(mask, dict):
                    raise ConfigError(f"config.json: {where}mixer.mask must be an object or null")
                window = take(mask, "size", int, None, positive=True) if mask else None
                keep = take(mask, "keep_first", int, 0) if mask else 0
                if keep < 0:
                    raise ConfigError(f"config.json: {where}mixer.mask.keep_first must not be negative")
                src = take(m, "kv_from", int, None)
                if src is not None:
                    if not (0 <= src < i) or raw[src].get("type") != "attention" or raw[src].get("mixer", {}).get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}mixer.kv_from = {src} must name an earlier attention layer "
                                          f"with keys and values of its own")
                mixer = DiffAttentionConfig(heads, kv, take(m, "dim", int, positive=True), take(m, "vdim", int, positive=True),
                                            take(m, "scale", float, positive=True), take(m, "diff", float), window, keep, src)
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not known (known: 'general_delta', 'attention')")
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"config.json: {where}mlp must be an object or null")
                if take(mlp, "kind", str) != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp['kind']!r} is not known (known: 'dense')")
                ff = take(mlp, "ff", int, positive=True)
            layers.append(ToriraxLayerConfig(kind, mixer, ff))
        for i, L in enumerate(layers):
            if L.type == "attention" and L.mixer.kv_from is not None:
                s, m = layers[L.mixer.kv_from].mixer, L.mixer
                if (s.kv_heads, s.dim, s.vdim) != (m.kv_heads, m.dim, m.vdim):
                    raise ConfigError(f"config.json: layers[{i}] reads the keys and values of layers[{m.kv_from}], whose "
                                      f"kv_heads, dim or vdim differ")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos)
        return cls(architecture=d["architectures"][0] if "architectures" in d else d["architecture"],
                   vocab=take(d, "vocab", int, positive=True), width=take(d, "width", int, positive=True),
                   max_positions=take(d, "max_positions", int, positive=True),
                   embedding_scale=take(_sub(d, "embedding", ""), "scale", float),
                   norm_eps=take(_sub(d, "norm", ""), "eps", float, positive=True), layers=tuple(layers),
                   eos_token_ids=eos_ids)

    def to_dict(self) -> Dict[str, Any]:
        d = dict(architecture=self.architecture, vocab=self.vocab, width=self.width, max_positions=self.max_positions,
                 embedding=dict(scale=self.embedding_scale), norm=dict(eps=self.norm_eps),
                 layers=[L.to_dict() for L in self.layers])
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
