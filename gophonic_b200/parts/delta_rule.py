"""The generalized delta rule as a mixer (``DeltaRuleSpec``): a matrix state per head that is decayed
per key channel, has the part along the token's unit key partly removed, and takes the token's k v^T.

One product projects x to r | k | v | g.  What enters the recurrence besides r, k and v is float32 from
the start: a second product, of the removal rate's matrix and the decay's first matrix together, leaves
float32; the decay's second product (after tanh) is float32 too, and the kernel of the recurrence turns the
pre-activations into factors in float32 (``ops.delta_scan``, state in the cache's per-sequence storage).  In a
step of single tokens that kernel forms the decay's second product itself, so the step runs no kernel between
the two projections and the recurrence.  Each head's output is divided by its root mean square, multiplied by
a weight and by sigmoid of the gate (``ops.head_norm_gate``), and projected back.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .base import Runtime, TensorDecl
from .linear_state import _StateMixer


class DeltaRule(_StateMixer):
    NAMES = ("r", "k", "v", "g")
    FUSED_ROWS = 16

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        kd, vd = spec.heads * spec.key_dim, spec.heads * spec.value_dim
        return [TensorDecl(prefix + "r", (kd, spec.hidden)), TensorDecl(prefix + "k", (kd, spec.hidden)),
                TensorDecl(prefix + "v", (vd, spec.hidden)), TensorDecl(prefix + "g", (vd, spec.hidden)),
                TensorDecl(prefix + "o", (spec.hidden, vd)),
                TensorDecl(prefix + "a", (kd, spec.hidden)), TensorDecl(prefix + "a.b", (kd,), role="vector"),
                TensorDecl(prefix + "w1", (spec.rank, spec.hidden)),      # rank None: whatever the checkpoint has
                TensorDecl(prefix + "w2", (kd, spec.rank)), TensorDecl(prefix + "w0", (kd,), role="vector"),
                TensorDecl(prefix + "norm", (vd,), role="norm")]

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        self.kd, self.vd = spec.heads * spec.key_dim, spec.heads * spec.value_dim
        mats = [tensors[prefix + n] for n in self.NAMES]
        if len({t.dtype for t in mats}) != 1:
            raise ValueError(f"{prefix}: the projections are stored in different dtypes; they must agree")
        self.qkvg = torch.cat(mats, dim=0).contiguous()      # r | k | v | g: one product reads x once
        self.o = tensors[prefix + "o"].contiguous()
        self.g_off = 2 * self.kd + self.vd
        a, w1 = tensors[prefix + "a"], tensors[prefix + "w1"]
        self.w2 = tensors[prefix + "w2"].contiguous()
        if w1.shape[0] != self.w2.shape[1]:
            raise ValueError(f"{prefix}: w1 has {w1.shape[0]} rows and w2 {self.w2.shape[1]} columns; they must agree")
        if a.dtype != w1.dtype:
            raise ValueError(f"{prefix}: a is {a.dtype} and w1 is {w1.dtype}; they must agree")
        self.rank = w1.shape[0]
        self.a_w1 = torch.cat([a, w1], dim=0).contiguous()       # the removal rate's rows, then the decay's first matrix: one float32 product
        self.a_bias = tensors[prefix + "a.b"].to(torch.float32).contiguous()
        self.w_bias = tensors[prefix + "w0"].to(torch.float32).contiguous()
        self.norm_w = tensors[prefix + "norm"].to(torch.float32).contiguous()

    def _matrices(self):
        return (self.qkvg, self.o, self.a_w1, self.w2)

    def _heads(self, batch, x: torch.Tensor, cache) -> torch.Tensor:
        """Everything up to the output projection: the normed and gated heads, [rows, heads * value_dim]."""
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        buf = self._project(x)
        both = torch.empty((rows, self.kd + self.rank), dtype=torch.float32, device=x.device)
        ops.gemm(x, self.a_w1, both)
        remove, low = both[:, :self.kd], both[:, self.kd:]
        o = torch.empty((rows, self.vd), dtype=torch.float32, device=x.device)
        decay = None
        # few single tokens: one kernel from the projections to the sums; many: the preparation kernel runs once a
        # (token, head) instead of once a CTA
        fused = batch.max_q_len == 1 and rows <= self.FUSED_ROWS and self.rank <= ops.DELTA_FUSED_MAX_RANK
        if not fused:
            ops.tanh_(low)
            decay = torch.empty((rows, self.kd), dtype=torch.float32, device=x.device)
            ops.gemm(low, self.w2, decay)
        ops.delta_scan(buf, 0, self.kd, 2 * self.kd, s.heads, s.key_dim, s.value_dim, decay, self.w_bias, float(s.decay_scale),
                       remove, self.a_bias, float(s.key_eps), cache.state, o, batch.seq_slot, batch.seq_q_start, batch.seq_q_len,
                       batch.nseq, max_q_len=batch.max_q_len, low=low if fused else None, w2=self.w2 if fused else None,
                       prepare=not fused)
        y = torch.empty((rows, self.vd), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(o, buf[:, self.g_off:self.g_off + self.vd], y, s.heads, s.value_dim, ops.GATE_SIGMOID,
                           weight=self.norm_w, eps=float(s.eps))
        return y
