"""What a layer adds to the stream at its end from the stream itself and the step's tokens.

``token_side``: a second embedding table holds, for every token, ``dim`` numbers for each layer of the model (a row is
``layers * dim`` long; a layer reads the columns from ``offset`` on).  With x the stream after the layer's last sublayer and
e the layer's slice of the token's row: ``g = gelu_tanh(W_gate x) * e`` (``W_gate`` is ``[dim, hidden]``), ``y = W_proj g``
(``[hidden, dim]``), and the stream takes ``y / sqrt(mean(y^2) + eps) * weight``.  The gate reads the stream, not a norm of it,
so the part first has the layer's pending delta added (one kernel, which also hands the stream on narrowed); the norm of y
and its addition are left to the next norm's kernel (a delta with ``post``).  Sums, the activation and the norm are float32.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import SIDES, Delta, PostNorm, SideInput, WeightDecl
from .linear import Linear


@SIDES.register("token_side")
class TokenSide(SideInput):
    NAMES = {"table": "side_embed.weight", "gate": "side_gate.weight", "proj": "side_proj.weight", "norm": "side_norm.weight"}

    def __init__(self, hidden: int, vocab: int, dim: int, table_cols: int, offset: int, eps: float, names: dict | None = None):
        self.hidden, self.vocab, self.dim = int(hidden), int(vocab), int(dim)
        self.table_cols, self.offset, self.eps = int(table_cols), int(offset), float(eps)
        if self.dim < 1 or self.offset < 0 or self.offset + self.dim > self.table_cols:
            raise ValueError(f"columns {offset} .. {offset + dim - 1} lie outside a table row of {table_cols} numbers")
        self.names = {**self.NAMES, **(names or {})}
        self.table: torch.Tensor | None = None
        self.gate: Linear | None = None
        self.proj: Linear | None = None
        self.norm: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        n = self.names
        return {n["table"]: WeightDecl((self.vocab, self.table_cols)), n["gate"]: WeightDecl((self.dim, self.hidden)),
                n["proj"]: WeightDecl((self.hidden, self.dim)), n["norm"]: WeightDecl((self.hidden,), init="norm")}

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        self.table = tensors[n["table"]].contiguous()
        self.gate, self.proj = Linear(tensors[n["gate"]]), Linear(tensors[n["proj"]])
        self.norm = tensors[n["norm"]].to(torch.float32).contiguous()

    def projections(self) -> list:
        return [self.gate, self.proj]

    def vectors(self) -> list[torch.Tensor]:
        return [self.norm]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, residual, pending: Delta | None) -> Delta:
        if pending is not None and (pending.post is not None or pending.depth is not None):
            raise RuntimeError("the token side input follows a plain delta")
        stream = ctx.scratch("side.stream", tuple(residual.shape))
        api.add_narrow(residual, None if pending is None else pending.tensor, stream)
        gated = ctx.scratch("side.gated", (ctx.n_tokens, self.dim))
        api.token_side_gate(self.gate(ctx, stream, "side.gate"), self.table, self.offset, ctx.tokens, gated, ctx.status)
        return Delta(self.proj(ctx, gated, "side.proj"), post=PostNorm(self.norm, self.eps, 0.0))
