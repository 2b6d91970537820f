"""Typed configuration of the Pugalix decoder, read from the keys of its ``config.json``.

A Pugalix model is a list of pre-norm layers, each with one mixer and an optional gated
feed-forward.  The file gives ``width``, ``vocab``, ``embedding.scale``, ``norm.eps`` and, per
entry of ``layers``, ``type`` (the mixer: ``attention``, ``gla`` or ``mlstm``), ``mixer`` (its sizes
and constants) and ``mlp`` (``{"kind": "dense", "ff": F}`` or null).  Tensor names are short:
``embed``, ``l<i>.norm1``, ``l<i>.mix.q`` (bias: ``l<i>.mix.q.b``), ``l<i>.mlp.gate``, ``final.norm``,
``head``.  Nothing but what the file says is assumed: every size and constant below comes from it
(the one size it does not carry, the rank of the decay projection of a ``gla`` mixer, is the shape
of that tensor; a file may name it as ``rank``, which random weights need).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .qwen3 import ConfigError
from .spec import (DecayStateSpec, EmbeddingSpec, GatedAttentionSpec, HeadSpec, LayerSpec, MatrixMemorySpec, ModelSpec,
                   PairRotarySpec, RMSNormSpec, ScheduleEntry, SwiGLUSpec)

_LIMIT = 16 << 20
MIXERS = ("attention", "gla", "mlstm")


def _get(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing key '{where}{key}'")
    return d[key]


def _int(d, key: str, where: str, low: int = 1) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{where}{key}' must be an integer, got {v!r}")
    if v < low or v > _LIMIT:
        raise ConfigError(f"config.json: '{where}{key}' = {v} is outside [{low}, {_LIMIT}]")
    return v


def _pos(d, key: str, where: str) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{where}{key}' must be a number, got {v!r}")
    v = float(v)
    if not (v > 0) or math.isinf(v):
        raise ConfigError(f"config.json: '{where}{key}' = {v} must be positive and finite")
    return v


@dataclass(frozen=True)
class PugalixLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]      # the mixer's keys, as read (nested dicts as tuples of pairs)
    ff: Optional[int]                       # width of the feed-forward, None: the layer has none

    def get(self, *path):
        node: Any = dict(self.mixer)
        for k in path:
            node = dict(node)[k]
        return node

    def has(self, key: str) -> bool:
        return key in dict(self.mixer)


def _freeze(v):
    if isinstance(v, dict):
        return tuple((k, _freeze(x)) for k, x in v.items())
    return v


def _thaw(v):
    if isinstance(v, tuple):
        return {k: _thaw(x) for k, x in v}
    return v


@dataclass(frozen=True)
class PugalixConfig:
    width: int
    vocab: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[PugalixLayer, ...]
    architecture: str = "Pugalix"

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PugalixConfig":
        width, vocab = _int(d, "width", ""), _int(d, "vocab", "")
        scale = _pos(d["embedding"], "scale", "embedding.") if isinstance(d.get("embedding"), dict) else 1.0
        eps = _pos(_get(d, "norm", ""), "eps", "norm.")
        raw_layers = _get(d, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[PugalixLayer] = []
        for i, raw in enumerate(raw_layers):
            at = f"layers[{i}]."
            kind = _get(raw, "type", at)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: '{at}type' is {kind!r}; this design has {', '.join(MIXERS)}")
            m = _get(raw, "mixer", at)
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: '{at}mixer' must be an object")
            ma = at + "mixer."
            m = dict(m)
            _int(m, "heads", ma), _int(m, "dim", ma)
            if m.get("vdim") is None:
                m["vdim"] = m["dim"]                 # values as wide as keys unless the file says otherwise
            _int(m, "vdim", ma)
            if kind == "attention":
                # what a file leaves out is not there: no grouping, no rotation, no window
                if m.get("kv_heads") is None:
                    m["kv_heads"] = m["heads"]
                if m.get("rot") is None:
                    m["rot"] = {"dims": 0, "base": 10000.0}
                if m.get("mask") is None:
                    m["mask"] = {"size": _LIMIT, "keep_first": 0}
                elif isinstance(m["mask"], dict) and m["mask"].get("keep_first") is None:
                    m["mask"] = dict(m["mask"], keep_first=0)
                heads, kvh = m["heads"], _int(m, "kv_heads", ma)
                if heads % kvh:
                    raise ConfigError(f"config.json: '{ma}heads' {heads} is not a multiple of '{ma}kv_heads' {kvh}")
                _pos(m, "scale", ma)
                rot, mask = _get(m, "rot", ma), _get(m, "mask", ma)
                dims = _int(rot, "dims", ma + "rot.", low=0)
                if dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"config.json: '{ma}rot.dims' {dims} must be even and at most '{ma}dim' {m['dim']}")
                _pos(rot, "base", ma + "rot.")
                _int(mask, "size", ma + "mask.")
                _int(mask, "keep_first", ma + "mask.", low=0)
                if m.get("kv_from") is not None:
                    j = _int(m, "kv_from", ma, low=0)
                    if j >= i or layers[j].type != "attention" or layers[j].has("kv_from"):
                        raise ConfigError(f"config.json: '{ma}kv_from' {j} must name an earlier attention layer with keys of its own")
                    src = layers[j]
                    same = (src.get("kv_heads") == kvh and src.get("dim") == m["dim"] and src.get("vdim") == m["vdim"]
                            and src.get("rot", "dims") == dims and float(src.get("rot", "base")) == float(rot["base"]))
                    if not same:
                        raise ConfigError(f"config.json: '{ma}kv_from' {j}: that layer's key/value heads or rotation differ")
            elif kind == "gla":
                _pos(m, "tau", ma)
                if m.get("rank") is not None:
                    _int(m, "rank", ma)
            else:
                _pos(m, "gate_cap", ma)
            mlp = raw.get("mlp") if isinstance(raw, dict) else None
            ff = None
            if mlp is not None:
                fk = _get(mlp, "kind", at + "mlp.")
                if fk != "dense":
                    raise ConfigError(f"config.json: '{at}mlp.kind' is {fk!r}; this design has dense feed-forwards")
                ff = _int(mlp, "ff", at + "mlp.")
            layers.append(PugalixLayer(kind, _freeze({k: v for k, v in m.items() if v is not None}), ff))
        return cls(width=width, vocab=vocab, embedding_scale=scale, norm_eps=eps, layers=tuple(layers),
                   architecture=str(d.get("architecture", "Pugalix")))

    # ---- writing -------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        return {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.type, "mixer": _thaw(l.mixer), "mlp": None if l.ff is None else {"ff": l.ff, "kind": "dense"}}
                       for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }

    def with_layers(self, n: int) -> "PugalixConfig":
        """The first ``n`` layers (a layer that takes its keys from a dropped layer cannot stay: layers are
        dropped from the end, so it never does)."""
        if not 0 < n <= len(self.layers):
            raise ValueError(f"layers={n} of a configuration with {len(self.layers)}")
        return PugalixConfig(self.width, self.vocab, self.embedding_scale, self.norm_eps, self.layers[:n], self.architecture)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    # ---- derived -------------------------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        layers, schedule = [], []
        for i, l in enumerate(self.layers):
            heads, d, dv = l.get("heads"), l.get("dim"), l.get("vdim")
            cache_of = None
            if l.type == "attention":
                cache_of = l.get("kv_from") if l.has("kv_from") else None
                mixer = GatedAttentionSpec(
                    hidden=W, heads=heads, kv_heads=l.get("kv_heads"), head_dim=d, value_dim=dv, scale=float(l.get("scale")),
                    position=PairRotarySpec(head_dim=d, rotary_dim=l.get("rot", "dims"), theta=float(l.get("rot", "base"))),
                    window=l.get("mask", "size"), keep_first=l.get("mask", "keep_first"), sink=True, bias=True, gate=True,
                    own_kv=cache_of is None)
            elif l.type == "gla":
                mixer = DecayStateSpec(hidden=W, heads=heads, key_dim=d, value_dim=dv, rank=l.get("rank") if l.has("rank") else None,
                                       tau=float(l.get("tau")), eps=eps)
            else:
                mixer = MatrixMemorySpec(hidden=W, heads=heads, key_dim=d, value_dim=dv, gate_cap=float(l.get("gate_cap")), eps=eps)
            ff = ff_norm = None
            if l.ff is not None:
                ff = SwiGLUSpec(hidden=W, intermediate=l.ff, names=("gate", "up", "down"))
                ff_norm = RMSNormSpec(size=W, eps=eps, tensor="")
            layers.append(LayerSpec(prefix=f"l{i}.", mixer=mixer, feed_forward=ff, mixer_norm=RMSNormSpec(size=W, eps=eps, tensor=""),
                                    feed_forward_norm=ff_norm, block="prenorm", mixer_prefix="mix.", feed_forward_prefix="mlp.",
                                    mixer_norm_prefix="norm1", feed_forward_norm_prefix="norm2"))
            schedule.append(ScheduleEntry(layer=i, cache_of=cache_of))
        spec = ModelSpec(
            architecture=self.architecture, hidden=W, vocab=self.vocab, max_positions=1 << 30,
            embedding=EmbeddingSpec("embed", self.vocab, W, scale=self.embedding_scale),
            layers=tuple(layers), schedule=tuple(schedule),
            final_norm=RMSNormSpec(size=W, eps=eps, tensor=""), final_norm_name="final.norm",
            head=HeadSpec("head", self.vocab, W, tied_to=None))
        spec.validate()
        return spec
