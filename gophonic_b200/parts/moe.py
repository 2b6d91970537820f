"""Mixture-of-experts feed-forward (``MoESpec``): every token uses the ``top`` experts its router scores
highest, out = sum over the chosen e of weight_e * down_e(relu(up_e x)^2).

The router's logits are a float32 product and its softmax, choice and weights are float32
(``ops.moe_route``).  The experts' matrices are kept stacked: all up matrices one above the other and all
down matrices side by side.  A step of many rows runs two products over the stack, with the row's weight
for each expert (zero where it was not chosen) folded into the activation between them, so the experts a
token did not choose contribute exact zeros and nothing depends on where the rows of an expert lie.  A
step of few rows reads only the chosen experts' matrices (``ops.moe_rows``).
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .base import FeedForward, Runtime, TensorDecl


class MoE(FeedForward):
    capturable = True
    ROWS_SPARSE = 16      # up to this many rows a step reads only the chosen experts' matrices

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
            ops.moe_rows(x, self.up, self.down, index, weight, out, s.experts, s.intermediate)
            return
        act = torch.empty((rows, s.experts * s.intermediate), dtype=x.dtype, device=x.device)
        ops.gemm(x, self.up, act)
        ops.moe_act(act, dense, act, s.experts, s.intermediate)
        ops.gemm(act, self.down, out)
