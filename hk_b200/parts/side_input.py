"""A per-layer token input: beside the model's embedding, a second table holds a short vector per token id and
layer, and every layer adds what it makes of its own slice to the residual stream:
    e = table[token][col0 : col0 + dim];   g = act(W_gate x) * e;   y = W_proj g;   x <- x + y / rms(y) * norm_weight
x is the residual stream as the layer's other sublayers left it (not normed).  The table is one tensor shared by
the layers (declared by each of them with the same name and shape); `col0`, `dim`, the activation and the eps are
parameters.  In a layer that runs several times every run reads the same slice."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import MATRIX, VECTOR, ParamSpec, Part, Precision, register_part


class TokenSideInput(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, hidden: int, vocab: int, table_name: str, table_cols: int, col0: int, dim: int, prefix: str, eps: float,
                 act: str = "gelu_tanh"):
        if col0 < 0 or col0 + dim > table_cols:
            raise ValueError(f"columns {col0}..{col0 + dim} are outside the table's {table_cols}")
        self.hidden, self.vocab, self.table_name, self.table_cols = hidden, vocab, table_name, int(table_cols)
        self.col0, self.dim, self.prefix, self.eps, self.act = int(col0), int(dim), prefix, float(eps), act
        self.table = self.w_gate = self.w_proj = self.norm_weight = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p = self.prefix
        return {
            self.table_name: ParamSpec((self.vocab, self.table_cols), MATRIX),
            p + "gate": ParamSpec((self.dim, self.hidden), MATRIX), p + "proj": ParamSpec((self.hidden, self.dim), MATRIX),
            p + "norm": ParamSpec((self.hidden,), VECTOR, "one_plus_normal"),
        }

    def own_bind(self, tensors, precision: Precision) -> None:
        p = self.prefix
        self.table = tensors[self.table_name]
        self.w_gate, self.w_proj, self.norm_weight = tensors[p + "gate"], tensors[p + "proj"], tensors[p + "norm"]

    def forward(self, residual: torch.Tensor, ctx) -> None:
        n = residual.shape[0]
        if self.w_gate.dtype == torch.float32:
            xb = residual
        else:
            xb = torch.empty(residual.shape, dtype=self.w_gate.dtype, device=residual.device)
            ops.narrow(residual, xb)
        z = torch.empty((n, self.dim), dtype=torch.float32, device=residual.device)
        ops.gemm(xb, self.w_gate, z)
        g = torch.empty((n, self.dim), dtype=self.w_proj.dtype, device=residual.device)
        ops.token_gate(z, self.table, self.col0, ctx.token_ids, g, self.act)
        y = torch.empty_like(residual)
        ops.gemm(g, self.w_proj, y)
        ops.rms_norm_add(y, self.norm_weight, self.eps, residual)


register_part("block", "token_side_input", TokenSideInput)
