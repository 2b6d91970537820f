"""Mixers that keep a matrix state per head instead of keys and values: gated linear attention
(``DecayState``) and the matrix memory of an mLSTM (``MatrixMemory``).

Both project x to q | k | v | g in one product, run the recurrence S <- diag(a) S + b k v^T,
o = S^T q token by token over the rows of a step (``ops.state_scan``, state in the cache's
per-sequence storage, float32), norm and gate the heads (``ops.head_norm_gate``) and project back.
What enters the recurrence besides q, k and v (decays, gates) comes out of a second, small product
in float32 and is turned into factors in float32.
"""
from __future__ import annotations

import math
from typing import List, Mapping

import torch

from .base import Mixer, Runtime, StateRequest, TensorDecl


class _StateMixer(Mixer):
    capturable = True

    @classmethod
    def _per_head(cls, spec) -> int:
        return spec.key_dim * spec.value_dim + cls.extra_state_of(spec)

    @classmethod
    def extra_state_of(cls, spec) -> int:
        return 0

    @classmethod
    def cache_request(cls, spec):
        return StateRequest(shape=(spec.heads, cls._per_head(spec)), dtype=torch.float32)

    def _common(self, spec, prefix, tensors, runtime):
        self.spec = spec
        self.rt = runtime
        self.kd, self.vd = spec.heads * spec.key_dim, spec.heads * spec.value_dim
        mats = [tensors[prefix + n] for n in ("q", "k", "v", "g")]
        if len({t.dtype for t in mats}) != 1:
            raise ValueError(f"{prefix}: the projections are stored in different dtypes; they must agree")
        self.qkvg = torch.cat(mats, dim=0).contiguous()
        self.o = tensors[prefix + "o"].contiguous()
        self.q_scale = 1.0 / math.sqrt(spec.key_dim)
        self.g_off = 2 * self.kd + self.vd

    @staticmethod
    def _common_decls(spec, prefix) -> List[TensorDecl]:
        kd, vd = spec.heads * spec.key_dim, spec.heads * spec.value_dim
        return [TensorDecl(prefix + "q", (kd, spec.hidden)), TensorDecl(prefix + "k", (kd, spec.hidden)),
                TensorDecl(prefix + "v", (vd, spec.hidden)), TensorDecl(prefix + "g", (vd, spec.hidden)),
                TensorDecl(prefix + "o", (spec.hidden, vd))]

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._matrices())

    # prompt-sized steps: the output projection adds into the float32 residual in its own epilogue
    def adds_in_place(self, rows: int) -> bool:
        ops = self.rt.ops
        return (self.o.dtype == torch.bfloat16 and self.rt.act_dtype == torch.bfloat16 and self.vd % 8 == 0
                and self.spec.hidden % 4 == 0 and ops.gemm_algo(rows, self.spec.hidden, self.vd) == "tc5_pair")

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor, cache) -> None:
        self.rt.ops.gemm(self._heads(batch, x, cache), self.o, out)

    def forward_into(self, batch, x: torch.Tensor, h: torch.Tensor, cache) -> None:
        self.rt.ops.gemm_add(self._heads(batch, x, cache), self.o, h)

    def _project(self, x):
        rows = x.shape[0]
        buf = torch.empty((rows, self.qkvg.shape[0]), dtype=x.dtype, device=x.device)
        self.rt.ops.gemm(x, self.qkvg, buf)
        return buf


class DecayState(_StateMixer):
    """Gated linear attention (``DecayStateSpec``)."""

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        kd = spec.heads * spec.key_dim
        return cls._common_decls(spec, prefix) + [
            TensorDecl(prefix + "norm", (spec.value_dim,), role="norm"),
            TensorDecl(prefix + "a1", (spec.rank, spec.hidden)),      # rank None: whatever the checkpoint has
            TensorDecl(prefix + "a2", (kd, spec.rank)),
            TensorDecl(prefix + "a2.b", (kd,), role="vector")]

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self._common(spec, prefix, tensors, runtime)
        self.a1, self.a2 = tensors[prefix + "a1"].contiguous(), tensors[prefix + "a2"].contiguous()
        if self.a1.shape[0] != self.a2.shape[1]:
            raise ValueError(f"{prefix}: a1 has {self.a1.shape[0]} rows and a2 {self.a2.shape[1]} columns; they must agree")
        self.a_bias = tensors[prefix + "a2.b"].to(torch.float32).contiguous()
        self.norm_w = tensors[prefix + "norm"].to(torch.float32).contiguous()

    def _matrices(self):
        return (self.qkvg, self.o, self.a1, self.a2)

    def _heads(self, batch, x: torch.Tensor, cache) -> torch.Tensor:
        """Everything up to the output projection: the normed and gated heads, [rows, heads * value_dim]."""
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        buf = self._project(x)
        # the decay's two small products leave float32; its bias, sigmoid and root are float32 too
        low = torch.empty((rows, self.a1.shape[0]), dtype=torch.float32, device=x.device)
        ops.gemm(x, self.a1, low)
        decay = torch.empty((rows, self.kd), dtype=torch.float32, device=x.device)
        ops.gemm(low, self.a2, decay)
        ops.gla_decay(decay, self.a_bias, float(s.tau))
        o = torch.empty((rows, self.vd), dtype=torch.float32, device=x.device)
        ops.state_scan(buf, 0, self.kd, 2 * self.kd, s.heads, s.key_dim, s.value_dim, self.q_scale, cache.state, o,
                       batch.seq_slot, batch.seq_q_start, batch.seq_q_len, batch.nseq, decay=decay, max_q_len=batch.max_q_len)
        y = torch.empty((rows, self.vd), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(o, buf[:, self.g_off:self.g_off + self.vd], y, s.heads, s.value_dim, ops.GATE_SILU,
                           weight=self.norm_w, eps=float(s.eps))
        return y


class MatrixMemory(_StateMixer):
    """The matrix memory of an mLSTM (``MatrixMemorySpec``)."""

    @classmethod
    def extra_state_of(cls, spec) -> int:
        # the normaliser and the running maximum, rounded up so that every head's matrix starts on 16 bytes
        return (spec.key_dim + 1 + 3) // 4 * 4

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        return cls._common_decls(spec, prefix) + [
            TensorDecl(prefix + "norm", (spec.heads * spec.value_dim,), role="norm"),
            TensorDecl(prefix + "i", (spec.heads, spec.hidden)), TensorDecl(prefix + "i.b", (spec.heads,), role="vector"),
            TensorDecl(prefix + "f", (spec.heads, spec.hidden)), TensorDecl(prefix + "f.b", (spec.heads,), role="vector")]

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self._common(spec, prefix, tensors, runtime)
        self.gates_w = torch.cat([tensors[prefix + "i"], tensors[prefix + "f"]], dim=0).contiguous()
        self.gate_bias = torch.cat([tensors[prefix + "i.b"], tensors[prefix + "f.b"]]).to(torch.float32).contiguous()
        self.norm_w = tensors[prefix + "norm"].to(torch.float32).contiguous()

    def _matrices(self):
        return (self.qkvg, self.o, self.gates_w)

    def _heads(self, batch, x: torch.Tensor, cache) -> torch.Tensor:
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        buf = self._project(x)
        gates = torch.empty((rows, 2 * s.heads), dtype=torch.float32, device=x.device)
        ops.gemm(x, self.gates_w, gates)
        coef = torch.empty((rows, s.heads, 4), dtype=torch.float32, device=x.device)
        o = torch.empty((rows, self.vd), dtype=torch.float32, device=x.device)
        ops.state_scan(buf, 0, self.kd, 2 * self.kd, s.heads, s.key_dim, s.value_dim, self.q_scale, cache.state, o,
                       batch.seq_slot, batch.seq_q_start, batch.seq_q_len, batch.nseq, gates=gates, gate_bias=self.gate_bias,
                       gate_cap=float(s.gate_cap), coef=coef, max_q_len=batch.max_q_len)
        y = torch.empty((rows, self.vd), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(o, buf[:, self.g_off:self.g_off + self.vd], y, s.heads, s.value_dim, ops.GATE_SIGMOID,
                           weight=self.norm_w, eps=float(s.eps), divisor=coef[:, :, 3:])
        return y
