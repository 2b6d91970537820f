"""The hyper-connection arrangement (``HyperLayerSpec``): the residual is S streams, a sublayer reads a
weighted sum of them and its output is spread over all of them while they are mixed.

For sublayer q (the mixer, then the feed-forward) with vectors in_q, out_q and a matrix mix_q ([from, to]):
u = sum_s in_q[s] x_s; y = sublayer(norm_q(u)); x_t <- sum_s mix_q[s, t] x_s + mult * out_q[t] * y for all t
from the old streams.  The streams are float32 throughout.  One row-wise kernel (``ops.hyper_mix_norm``)
does the spreading of one sublayer's output and the read and norm for the next sublayer in one pass over
the streams, also across the border between two layers: the block hands its last sublayer's output on as
the pending addend, with itself as the one who knows how to add it, and the next block (or the model's
final norm) adds it while it reads.  With ``streams`` 0 the same code is the plain residual
x <- x + mult * y: one stream, no tensors.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Mapping, Optional

import torch

from .. import registry
from .base import Part, Runtime, TensorDecl


@dataclass
class PendingSpread:
    """A sublayer's output that has yet to be spread over the streams, and the coefficients to do it with."""
    y: torch.Tensor
    mix: Optional[torch.Tensor]
    out: Optional[torch.Tensor]
    mult: float


class HyperBlock(Part):
    category = "block"
    takes_streams = True     # forward gets the residual as [streams, rows, hidden]

    @classmethod
    def declare(cls, layer, prefix: str = "") -> List[TensorDecl]:
        p = layer.prefix
        decls: List[TensorDecl] = []
        decls += registry.part_class("norm", layer.mixer_norm.kind).declare(layer.mixer_norm, p + layer.mixer_norm_prefix)
        decls += registry.part_class("mixer", layer.mixer.kind).declare(layer.mixer, p + layer.mixer_prefix)
        if layer.feed_forward is not None:
            decls += registry.part_class("norm", layer.feed_forward_norm.kind).declare(
                layer.feed_forward_norm, p + layer.feed_forward_norm_prefix)
            decls += registry.part_class("feed_forward", layer.feed_forward.kind).declare(
                layer.feed_forward, p + layer.feed_forward_prefix)
        S = layer.streams
        if S > 0:
            for q in range(2 if layer.feed_forward is not None else 1):
                c = p + layer.connection_prefixes[q]
                decls += [TensorDecl(c + "in", (S,), role="norm"), TensorDecl(c + "out", (S,), role="norm"),
                          TensorDecl(c + "mix", (S, S), role="identity")]
        return decls

    def __init__(self, layer, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        p = layer.prefix
        self.layer = layer
        self.rt = runtime
        self.mult = float(layer.residual_mult)
        self.mixer_norm = registry.part_class("norm", layer.mixer_norm.kind)(
            layer.mixer_norm, p + layer.mixer_norm_prefix, tensors, runtime)
        self.mixer = registry.part_class("mixer", layer.mixer.kind)(layer.mixer, p + layer.mixer_prefix, tensors, runtime)
        self.feed_forward_norm = self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = registry.part_class("norm", layer.feed_forward_norm.kind)(
                layer.feed_forward_norm, p + layer.feed_forward_norm_prefix, tensors, runtime)
            self.feed_forward = registry.part_class("feed_forward", layer.feed_forward.kind)(
                layer.feed_forward, p + layer.feed_forward_prefix, tensors, runtime)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and norm.rms_fold() is None:
                raise ValueError(f"{p}: the hyper-connection block reads its streams through an RMS norm with a weight")
        # (in, out, mix) of each sublayer, float32; None: ones and the identity
        self.connections = []
        for q in range(2):
            c = p + layer.connection_prefixes[q]
            if layer.streams > 0 and (q == 0 or layer.feed_forward is not None):
                self.connections.append(tuple(tensors[c + n].to(torch.float32).contiguous() for n in ("in", "out", "mix")))
            else:
                self.connections.append((None, None, None))

    @classmethod
    def cache_request(cls, layer):
        return registry.part_class("mixer", layer.mixer.kind).cache_request(layer.mixer)

    def prepare(self, capacity: int) -> None:
        self.mixer.prepare(capacity)

    def mixers(self) -> List[Part]:
        return [self.mixer]

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.mixer, self.feed_forward) if p is not None and hasattr(p, "weight_bytes"))

    @property
    def capturable(self) -> bool:
        return all(p.capturable for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None)

    def _read(self, streams: torch.Tensor, pending, q: int, norm) -> torch.Tensor:
        """Spread what is pending over the streams and read them for sublayer ``q``: the normed input."""
        rows, hidden = streams.shape[1], streams.shape[2]
        x = torch.empty((rows, hidden), dtype=self.rt.act_dtype, device=streams.device)
        weight, eps = norm.rms_fold()
        kw = {}
        if pending is not None:
            kw = dict(y=pending.y, mix=pending.mix, out_coef=pending.out, mult=pending.mult)
        self.rt.ops.hyper_mix_norm(streams, in_coef=self.connections[q][0], norm_weight=weight, eps=eps, x_out=x, **kw)
        return x

    def forward(self, batch, streams: torch.Tensor, pending, cache):
        """Runs the layer on the residual ``streams`` (float32 [S, rows, hidden], updated in place).
        ``pending``: a ``PendingSpread`` the block before left (its last sublayer's output, not yet spread
        over the streams) or None.  Returns the ``PendingSpread`` of this block's last sublayer."""
        if pending is not None and not isinstance(pending, PendingSpread):
            raise TypeError("a hyper-connection block follows only blocks of its own kind")
        rows, hidden = streams.shape[1], streams.shape[2]
        x = self._read(streams, pending, 0, self.mixer_norm)
        y = torch.empty((rows, hidden), dtype=torch.float32, device=streams.device)
        self.mixer.forward(batch, x, y, cache)
        pending = PendingSpread(y, self.connections[0][2], self.connections[0][1], self.mult)
        if self.feed_forward is None:
            return pending
        x = self._read(streams, pending, 1, self.feed_forward_norm)
        y = torch.empty((rows, hidden), dtype=torch.float32, device=streams.device)
        self.feed_forward.forward(batch, x, y)
        return PendingSpread(y, self.connections[1][2], self.connections[1][1], self.mult)

    def finish(self, streams: torch.Tensor, pending, norm, x_out: torch.Tensor, rows: Optional[torch.Tensor]) -> None:
        """The model's last step: spread what is pending, then x_out = norm(sum of the streams) for the
        wanted rows."""
        ops = self.rt.ops
        weight, eps = norm.rms_fold()
        kw = {}
        if pending is not None:
            kw = dict(y=pending.y, mix=pending.mix, out_coef=pending.out, mult=pending.mult)
        ops.hyper_mix_norm(streams, norm_weight=weight, eps=eps, x_out=x_out, rows=rows, **kw)
