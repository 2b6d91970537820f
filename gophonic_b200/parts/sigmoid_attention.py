"""Grouped-query attention with sigmoid weights (``SigmoidAttentionSpec``): a visible key weighs
sigmoid(score + a bias per head), nothing is normalised over the keys.

Per row: q | k | v | g = x [Wq; Wk; Wv; Wg]^T in one product (g: one gate pre-activation per head); a short
causal convolution over time on every channel of q, k and v, each head of q, k and v over its root mean
square, q into a buffer and k, v into the cache, in one row-wise kernel that reaches back into the
sequence's last projected rows (``ops.conv_qkv``: they are the fixed-size part of this mixer's cache, beside
its keys and values); scores (q . k) * scale in float32 over the keys j <= i inside the window; the heads,
each ``value_dim`` wide, times sigmoid of their gate; out = ctx Wo^T.  No position enters the scores.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .base import KVRequest, KVStateRequest, Mixer, Runtime, StateRequest, TensorDecl


class SigmoidAttention(Mixer):
    capturable = True

    @staticmethod
    def _dims(spec):
        return spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim, spec.kv_heads * spec.value_dim, spec.heads * spec.value_dim

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        qd, kd, vd, od = cls._dims(spec)
        decls = [TensorDecl(prefix + "q", (qd, spec.hidden)), TensorDecl(prefix + "k", (kd, spec.hidden)),
                 TensorDecl(prefix + "v", (vd, spec.hidden)), TensorDecl(prefix + "o", (spec.hidden, od))]
        if spec.conv_taps > 0:
            decls += [TensorDecl(prefix + n + ".conv", (size, spec.conv_taps)) for n, size in (("q", qd), ("k", kd), ("v", vd))]
        if spec.score_bias:
            decls.append(TensorDecl(prefix + "pb", (spec.heads,), role="vector"))
        if spec.head_gate:
            decls.append(TensorDecl(prefix + "g", (spec.heads, spec.hidden)))
        return decls

    @classmethod
    def cache_request(cls, spec):
        # every key is kept (the window is a mask)
        kv = KVRequest(kv_heads=spec.kv_heads, head_dim=spec.head_dim, window=0, value_dim=spec.value_dim)
        if spec.conv_taps <= 1:
            return kv
        qd, kd, vd, _ = cls._dims(spec)
        return KVStateRequest(kv, StateRequest(shape=((spec.conv_taps - 1) * (qd + kd + vd),), dtype=torch.float32))

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        if spec.heads % spec.kv_heads:
            raise ValueError(f"{prefix}: {spec.heads} heads are not a multiple of {spec.kv_heads} kv heads")
        self.spec = spec
        self.rt = runtime
        self.q_dim, self.k_dim, self.v_dim, self.o_dim = self._dims(spec)
        parts = [tensors[prefix + "q"], tensors[prefix + "k"], tensors[prefix + "v"]]
        if spec.head_gate:
            parts.append(tensors[prefix + "g"])
        if len({t.dtype for t in parts}) != 1:
            raise ValueError(f"{prefix}: the projections are stored in different dtypes; they must agree")
        rows = sum(t.shape[0] for t in parts)
        pad = (-rows) % 8           # rows of the product's output stay 16-byte aligned for the kernels that read them
        if pad:
            parts.append(torch.zeros((pad, spec.hidden), dtype=parts[0].dtype, device=parts[0].device))
        self.qkvg = torch.cat(parts, dim=0).contiguous()
        self.g_off = self.q_dim + self.k_dim + self.v_dim
        self.o = tensors[prefix + "o"].contiguous()
        self.conv = None
        if spec.conv_taps > 0:
            self.conv = torch.cat([tensors[prefix + n + ".conv"] for n in ("q", "k", "v")], dim=0).to(torch.float32).contiguous()
        self.score_bias = tensors[prefix + "pb"].to(torch.float32).contiguous() if spec.score_bias else None

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.qkvg, self.o))

    # prompt-sized steps: the output projection adds into a float32 buffer in its own epilogue
    def adds_in_place(self, rows: int) -> bool:
        ops = self.rt.ops
        return (self.o.dtype == torch.bfloat16 and self.rt.act_dtype == torch.bfloat16 and self.o_dim % 8 == 0
                and self.spec.hidden % 4 == 0 and ops.gemm_algo(rows, self.spec.hidden, self.o_dim) == "tc5_pair")

    def forward_into(self, batch, x: torch.Tensor, h: torch.Tensor, cache) -> None:
        self.rt.ops.gemm_add(self._gated_heads(batch, x, cache), self.o, h)

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor, cache) -> None:
        self.rt.ops.gemm(self._gated_heads(batch, x, cache), self.o, out)

    def _gated_heads(self, batch, x: torch.Tensor, cache) -> torch.Tensor:
        """Everything up to the output projection: [rows, heads * value_dim] in the activation dtype."""
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        if cache is None or not cache.writable:
            raise ValueError("attention needs a key/value cache plane of its own")
        if cache.k.dtype != x.dtype:
            raise ValueError(f"attention: cache holds {cache.k.dtype}, activations are {x.dtype}")
        qkvg = torch.empty((rows, self.qkvg.shape[0]), dtype=x.dtype, device=x.device)
        ops.gemm(x, self.qkvg, qkvg)
        q = torch.empty((rows, self.q_dim), dtype=x.dtype, device=x.device)
        ops.conv_qkv(qkvg, q, s.heads, s.kv_heads, s.head_dim, s.value_dim, self.conv, cache.state, bool(s.qk_norm), bool(s.v_norm),
                     float(s.eps), batch, cache.block_table, cache.k, cache.v)
        ctx = torch.empty((rows, self.o_dim), dtype=x.dtype, device=x.device)
        gate = qkvg[:, self.g_off:self.g_off + s.heads] if s.head_gate else None
        ops.attention_sigmoid(q, ctx, cache.k, cache.v, cache.block_table, batch, s.heads, s.kv_heads, s.head_dim, float(s.scale),
                              int(s.window), value_dim=s.value_dim, score_bias=self.score_bias, gate=gate)
        return ctx
