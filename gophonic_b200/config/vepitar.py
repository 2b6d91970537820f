"""Typed configuration of the Vepitar decoder, read from the keys of its ``config.json``.

A Vepitar model is a list of pre-norm layers whose residual may be kept in several streams
(hyper-connections).  The file gives ``width``, ``vocab``, ``norm.eps``, ``residual_mult`` (the factor
on every sublayer's output; 1 if absent), ``streams`` (absent: one plain residual) and, per entry of
``layers``, ``type`` (the mixer: ``general_delta`` or ``attention``), ``mixer`` (its sizes and constants)
and ``mlp``: ``{"kind": "dense", "ff": F}``, ``{"kind": "moe", "expert": {"ff": F}, "router": {"experts": E,
"top": K}}`` or null.  A norm's tensor holds its weight's difference from one (the norm multiplies by 1 + w) and the head is
the embedding table.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.q`` (its convolution:
``l<i>.mix.q.conv``), ``l<i>.mlp.gate``, ``l<i>.mlp.e<j>.up``, ``l<i>.mlp.router``, ``l<i>.hc1.in``,
``final.norm``.  What the file leaves out is not there: an attention mixer without ``conv`` has no
convolution, without ``mask`` no window, without ``kv_heads`` as many key heads as query heads, without
``vdim`` values as wide as keys.  The one size the file does not carry, the rank of the decay projection
of a ``general_delta`` mixer, is the shape of that tensor (a file may name it as ``rank``, which random
weights need).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .pugalix import _LIMIT, _freeze, _get, _int, _pos, _thaw
from .qwen3 import ConfigError
from .spec import (DeltaRuleSpec, EmbeddingSpec, HeadSpec, HyperLayerSpec, ModelSpec, MoESpec, RMSNormSpec, ScheduleEntry,
                   SigmoidAttentionSpec, SwiGLUSpec)

MIXERS = ("general_delta", "attention")
MAX_STREAMS = 8
# constants the design fixes
DELTA_DECAY_SCALE = math.exp(-0.5)     # the decay is exp(-DELTA_DECAY_SCALE * sigmoid(.))
DELTA_KEY_EPS = 1e-6                   # under the root of the unit key's length
MOE_RENORM_EPS = 1e-20                 # added to the sum of the chosen scores


@dataclass(frozen=True)
class VepitarLayer:
    type: str
    mixer: Tuple[Tuple[str, Any], ...]      # the mixer's keys, as read (nested dicts as tuples of pairs)
    mlp: Optional[Tuple[Tuple[str, Any], ...]]

    def get(self, *path):
        node: Any = dict(self.mixer)
        for k in path:
            node = dict(node)[k]
        return node

    def has(self, key: str) -> bool:
        return key in dict(self.mixer)


@dataclass(frozen=True)
class VepitarConfig:
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    streams: Optional[int]                  # None: one plain residual, no connection tensors
    layers: Tuple[VepitarLayer, ...]
    architecture: str = "Vepitar"
    tie_word_embeddings = True              # the head is the embedding table

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VepitarConfig":
        width, vocab = _int(d, "width", ""), _int(d, "vocab", "")
        eps = _pos(_get(d, "norm", ""), "eps", "norm.")
        mult = 1.0
        if d.get("residual_mult") is not None:
            mult = d["residual_mult"]
            if isinstance(mult, bool) or not isinstance(mult, (int, float)) or not math.isfinite(float(mult)):
                raise ConfigError(f"config.json: 'residual_mult' must be a finite number, got {mult!r}")
            mult = float(mult)
        streams = None
        if d.get("streams") is not None:
            streams = _int(d, "streams", "")
            if streams > MAX_STREAMS:
                raise ConfigError(f"config.json: 'streams' = {streams}; at most {MAX_STREAMS}")
        raw_layers = _get(d, "layers", "")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[VepitarLayer] = []
        for i, raw in enumerate(raw_layers):
            at = f"layers[{i}]."
            kind = _get(raw, "type", at)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: '{at}type' is {kind!r}; this design has {', '.join(MIXERS)}")
            m = _get(raw, "mixer", at)
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: '{at}mixer' must be an object")
            ma = at + "mixer."
            m = {k: v for k, v in m.items() if v is not None}
            _int(m, "heads", ma), _int(m, "dim", ma)
            if "vdim" in m:
                _int(m, "vdim", ma)
            if kind == "attention":
                if "kv_heads" in m and m["heads"] % _int(m, "kv_heads", ma):
                    raise ConfigError(f"config.json: '{ma}heads' {m['heads']} is not a multiple of '{ma}kv_heads' {m['kv_heads']}")
                _pos(m, "scale", ma)
                if "mask" in m:
                    _int(_get(m, "mask", ma), "size", ma + "mask.")
                if "conv" in m:
                    _int(m, "conv", ma)
            elif "rank" in m:
                _int(m, "rank", ma)
            mlp = raw.get("mlp") if isinstance(raw, dict) else None
            if mlp is not None:
                fk = _get(mlp, "kind", at + "mlp.")
                if fk == "dense":
                    _int(mlp, "ff", at + "mlp.")
                elif fk == "moe":
                    _int(_get(mlp, "expert", at + "mlp."), "ff", at + "mlp.expert.")
                    router = _get(mlp, "router", at + "mlp.")
                    experts, top = _int(router, "experts", at + "mlp.router."), _int(router, "top", at + "mlp.router.")
                    if top > experts:
                        raise ConfigError(f"config.json: '{at}mlp.router.top' {top} exceeds its {experts} experts")
                else:
                    raise ConfigError(f"config.json: '{at}mlp.kind' is {fk!r}; this design has dense and moe feed-forwards")
            layers.append(VepitarLayer(kind, _freeze(m), None if mlp is None else _freeze(dict(mlp))))
        return cls(width=width, vocab=vocab, norm_eps=eps, residual_mult=mult, streams=streams, layers=tuple(layers),
                   architecture=str(d.get("architecture", "Vepitar")))

    # ---- writing -------------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        out = {
            "architecture": self.architecture,
            "layers": [{"type": l.type, "mixer": _thaw(l.mixer), "mlp": None if l.mlp is None else _thaw(l.mlp)} for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.streams is not None:
            out["streams"] = self.streams
        return out

    def with_layers(self, n: int) -> "VepitarConfig":
        if not 0 < n <= len(self.layers):
            raise ValueError(f"layers={n} of a configuration with {len(self.layers)}")
        return VepitarConfig(self.width, self.vocab, self.norm_eps, self.residual_mult, self.streams, self.layers[:n], self.architecture)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    # ---- derived -------------------------------------------------------------------------
    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = lambda: RMSNormSpec(size=W, eps=eps, tensor="", offset=1.0)
        layers, schedule = [], []
        for i, l in enumerate(self.layers):
            heads, d = l.get("heads"), l.get("dim")
            dv = l.get("vdim") if l.has("vdim") else d
            if l.type == "attention":
                mixer = SigmoidAttentionSpec(
                    hidden=W, heads=heads, kv_heads=l.get("kv_heads") if l.has("kv_heads") else heads, head_dim=d, value_dim=dv,
                    scale=float(l.get("scale")), window=l.get("mask", "size") if l.has("mask") else 0,
                    conv_taps=l.get("conv") if l.has("conv") else 0, eps=eps)
            else:
                mixer = DeltaRuleSpec(hidden=W, heads=heads, key_dim=d, value_dim=dv, rank=l.get("rank") if l.has("rank") else None,
                                      decay_scale=DELTA_DECAY_SCALE, key_eps=DELTA_KEY_EPS, eps=eps)
            ff = ff_norm = None
            if l.mlp is not None:
                mlp = _thaw(l.mlp)
                if mlp["kind"] == "dense":
                    ff = SwiGLUSpec(hidden=W, intermediate=mlp["ff"], names=("gate", "up", "down"))
                else:
                    ff = MoESpec(hidden=W, experts=mlp["router"]["experts"], top=mlp["router"]["top"], intermediate=mlp["expert"]["ff"],
                                 renorm_eps=MOE_RENORM_EPS)
                ff_norm = norm()
            layers.append(HyperLayerSpec(prefix=f"l{i}.", mixer=mixer, feed_forward=ff, mixer_norm=norm(), feed_forward_norm=ff_norm,
                                         streams=self.streams or 0, residual_mult=self.residual_mult))
            schedule.append(ScheduleEntry(layer=i))
        spec = ModelSpec(
            architecture=self.architecture, hidden=W, vocab=self.vocab, max_positions=1 << 30,
            embedding=EmbeddingSpec("embed", self.vocab, W), layers=tuple(layers), schedule=tuple(schedule),
            final_norm=norm(), final_norm_name="final.norm", head=HeadSpec("head", self.vocab, W, tied_to="embed"),
            streams=self.streams or 1)
        spec.validate()
        return spec
