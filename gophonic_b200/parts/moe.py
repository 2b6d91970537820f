"""Mixture-of-experts feed-forward (``MoESpec``): every token uses the ``top`` experts its router scores
highest, out = sum over the chosen e of weight_e * down_e(relu(up_e x)^2).

The router's logits are a float32 product and its softmax, choice and weights are float32
(``ops.moe_route``).  The experts' matrices are kept stacked: all up matrices one above the other and all
down matrices side by side.  A step of many rows runs two products over the stack, with the row's weight
for each expert (zero where it was not chosen) folded into the activation between them, so the experts a
token did not choose contribute exact zeros and nothing depends on where the rows of an expert lie; such
a step stays free of host reads, so single-token steps of many sequences replay from a graph.  A step of
few rows reads only the chosen experts' matrices (``ops.moe_rows``; with more (row, choice) pairs than
experts the pairs are sorted by expert on the device first, so that an expert's matrices are read once:
``ops.moe_rows_grouped``).  A prompt-sized step, which is never
replayed from a graph, sorts its (row, choice) pairs by expert, reads the experts' group sizes on the host
and runs one pair of products an expert on that expert's rows alone, so it does top / experts of the stacked
path's arithmetic.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .base import FeedForward, Runtime, TensorDecl


class MoE(FeedForward):
    capturable = True
    ROWS_SPARSE = 16      # up to this many rows a step reads only the chosen experts' matrices
    ROWS_GROUPED = 192    # from this many rows on a step runs every expert on its own rows (it reads their counts on the host)

    @classmethod
    def declare(cls, spec, prefix: str) -> List[TensorDecl]:
        decls = [TensorDecl(prefix + "router", (spec.experts, spec.hidden))]
        for e in range(spec.experts):
            decls += [TensorDecl(prefix + f"e{e}.up", (spec.intermediate, spec.hidden)),
                      TensorDecl(prefix + f"e{e}.down", (spec.hidden, spec.intermediate))]
        return decls

    def __init__(self, spec, prefix: str, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.rt = runtime
        ups = [tensors[prefix + f"e{e}.up"] for e in range(spec.experts)]
        downs = [tensors[prefix + f"e{e}.down"] for e in range(spec.experts)]
        if len({t.dtype for t in ups + downs}) != 1:
            raise ValueError(f"{prefix}: the experts are stored in different dtypes; they must agree")
        self.up = torch.cat(ups, dim=0).contiguous()         # [experts * ff, hidden]
        self.down = torch.cat(downs, dim=1).contiguous()     # [hidden, experts * ff]
        self.router = tensors[prefix + "router"].contiguous()

    def weight_bytes(self) -> int:
        """Bytes of the matrices a token's step reads: the router and the chosen experts."""
        per = (self.up.numel() + self.down.numel()) * self.up.element_size() // self.spec.experts
        return self.router.numel() * self.router.element_size() + per * self.spec.top

    def forward(self, batch, x: torch.Tensor, out: torch.Tensor) -> None:
        ops, s = self.rt.ops, self.spec
        rows = x.shape[0]
        logits = torch.empty((rows, s.experts), dtype=torch.float32, device=x.device)
        ops.gemm(x, self.router, logits)
        dense = torch.empty((rows, s.experts), dtype=torch.float32, device=x.device)
        index = torch.empty((rows, s.top), dtype=torch.int32, device=x.device)
        weight = torch.empty((rows, s.top), dtype=torch.float32, device=x.device)
        ops.moe_route(logits, s.top, float(s.renorm_eps), dense, index, weight)
        if rows <= self.ROWS_SPARSE and s.top < s.experts:
            if rows * s.top <= s.experts:      # hardly two pairs with one expert: a pair reads its expert's matrices
                ops.moe_rows(x, self.up, self.down, index, weight, out, s.experts, s.intermediate)
                return
            # more pairs than experts: sorted by expert on the device, every expert's matrices are read once
            pairs = rows * s.top
            offsets = torch.empty(s.experts + 1, dtype=torch.int32, device=x.device)
            place = torch.empty(pairs, dtype=torch.int32, device=x.device)
            src_row = torch.empty(pairs, dtype=torch.int32, device=x.device)
            ops.moe_group(index, s.experts, offsets, place, src_row)
            ys = torch.empty((pairs, s.hidden), dtype=torch.float32, device=x.device)
            ops.moe_rows_grouped(x, self.up, self.down, offsets, src_row, ys, s.experts, s.top, s.intermediate)
            ops.moe_combine(ys, place, weight, out)
            return
        if rows >= self.ROWS_GROUPED and s.top < s.experts and not torch.cuda.is_current_stream_capturing():
            self._grouped(x, index, weight, out)
            return
        act = torch.empty((rows, s.experts * s.intermediate), dtype=x.dtype, device=x.device)
        ops.gemm(x, self.up, act)
        ops.moe_act(act, dense, act, s.experts, s.intermediate)
        ops.gemm(act, self.down, out)

    def _grouped(self, x: torch.Tensor, index: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
        """Every expert on its own rows: sort the pairs by expert, gather, two products an expert, add up."""
        ops, s = self.rt.ops, self.spec
        rows, pairs, ff = x.shape[0], x.shape[0] * s.top, s.intermediate
        offsets = torch.empty(s.experts + 1, dtype=torch.int32, device=x.device)
        place = torch.empty(pairs, dtype=torch.int32, device=x.device)
        src_row = torch.empty(pairs, dtype=torch.int32, device=x.device)
        ops.moe_group(index, s.experts, offsets, place, src_row)
        bounds = offsets.tolist()               # the one host read of a prompt-sized step
        xs = torch.empty((pairs, s.hidden), dtype=x.dtype, device=x.device)
        ops.moe_gather(x, src_row, xs)
        act = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
        for e in range(s.experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                ops.gemm_w_cols(xs[lo:hi], self.up[e * ff:(e + 1) * ff], act[lo:hi])
        ops.relu2(act)
        ys = torch.empty((pairs, s.hidden), dtype=torch.float32, device=x.device)
        for e in range(s.experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                ops.gemm_w_cols(act[lo:hi], self.down[:, e * ff:(e + 1) * ff], ys[lo:hi])
        ops.moe_combine(ys, place, weight, out)
