"""Token embedding and output head.

``h0 = E[token] * scale`` with scale 1 for Llama (thinruntime/gpu_runtime.py:10072,
thinruntime/model_arch.py:234-238).  The head is ``lm_head.weight`` when the checkpoint
has one and the embedding table otherwise (thinruntime/gpu_runtime.py:10395-10401);
logits are float32.  Two more embeddings add a second row to the token's: one chosen by the pair of the
previous token and this one, one by the token's position.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import EMBEDDINGS, HEADS, Embedding, Head, StateNeed, WeightDecl
from .linear import Linear


@EMBEDDINGS.register("table")
class TokenEmbedding(Embedding):
    def __init__(self, vocab: int, hidden: int, scale: float = 1.0, name: str = "weight"):
        self.vocab, self.hidden, self.scale = int(vocab), int(hidden), float(scale)
        self.name = name                        # what the checkpoint calls the table, behind the part's prefix
        self.table: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        return {self.name: WeightDecl((self.vocab, self.hidden))}

    def bind(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name].contiguous()

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, tokens, residual, states=None) -> None:
        api.embed_gather(self.table, tokens, residual, self.scale, ctx.status)


@EMBEDDINGS.register("table_positions")
class PositionedEmbedding(TokenEmbedding):
    """The token's row plus a learned vector of the token's position: ``h0 = E[token] * scale + P[position]`` with
    ``positions`` rows in ``P``; positions count from 0 in each sequence.  A token at a position beyond the table raises
    the status word's bad-token bit (its row is zero); the engine refuses such a step beforehand (``max_positions``)."""

    def __init__(self, vocab: int, hidden: int, positions: int, scale: float = 1.0, name: str = "weight", position_name: str = "positions.weight"):
        super().__init__(vocab, hidden, scale, name)
        self.max_positions = int(positions)
        self.position_name = position_name
        self.position_table: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        return {**super().weights(), self.position_name: WeightDecl((self.max_positions, self.hidden))}

    def bind(self, tensors, dtype, device) -> None:
        super().bind(tensors, dtype, device)
        self.position_table = tensors[self.position_name].to(self.table.dtype).contiguous()

    def forward(self, ctx, tokens, residual, states=None) -> None:
        api.embed_position_gather(self.table, self.position_table, tokens, ctx.cu, ctx.len_before, ctx.sequences, residual, self.scale,
                                  ctx.status)


@EMBEDDINGS.register("table_pair_hash")
class PairHashEmbedding(TokenEmbedding):
    """The token's row plus a row of a second table chosen by the pair (previous token, token):
    ``h0 = E[token] * scale + P[(previous * mul_prev + token * mul_cur) mod buckets]``, and ``P[buckets]`` (the last row)
    for a sequence's first token.  The previous token is a per-sequence state (int32, the token plus one; zero: none yet),
    so prompts cut into steps and decoding continue where the sequence stands."""

    def __init__(self, vocab: int, hidden: int, buckets: int, mul_prev: int, mul_cur: int, scale: float = 1.0, name: str = "weight",
                 pair_name: str = "pair.weight"):
        super().__init__(vocab, hidden, scale, name)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        if self.buckets < 1 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("the pair table needs at least one bucket and multipliers that are not negative")
        self.pair_name = pair_name
        self.pair_table: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        return {**super().weights(), self.pair_name: WeightDecl((self.buckets + 1, self.hidden))}

    def state_needs(self) -> list[StateNeed]:
        return [StateNeed((), torch.int32)]

    def bind(self, tensors, dtype, device) -> None:
        super().bind(tensors, dtype, device)
        self.pair_table = tensors[self.pair_name].to(self.table.dtype).contiguous()

    def forward(self, ctx, tokens, residual, states=None) -> None:
        if not states:
            raise RuntimeError("the pair embedding needs its per-sequence state (the previous token)")
        api.embed_pair_gather(self.table, self.pair_table, tokens, ctx.cu, ctx.slots, ctx.sequences, states[0], residual, self.buckets,
                              self.mul_prev, self.mul_cur, self.scale, ctx.status)


@HEADS.register("linear")
class LinearHead(Head):
    """``fallback`` is the checkpoint name of the tensor that serves as the head when
    the checkpoint stores none (the embedding table); with ``tied`` it is used even if
    a head is stored.  ``scale`` multiplies the logits."""

    def __init__(self, hidden: int, vocab: int, fallback: str | None = None, tied: bool = False, bias: bool = False,
                 name: str = "weight", scale: float = 1.0):
        self.hidden, self.vocab, self.fallback, self.tied, self.bias = int(hidden), int(vocab), fallback, bool(tied), bool(bias)
        self.name = name
        self.scale = float(scale)                # the logits are multiplied by it
        self.linear: Linear | None = None

    def weights(self) -> dict[str, WeightDecl]:
        out = {self.name: WeightDecl((self.vocab, self.hidden), alias_of=self.fallback, prefer_alias=self.tied)}
        if self.bias:
            out["bias"] = WeightDecl((self.vocab,))
        return out

    def bind(self, tensors, dtype, device) -> None:
        self.linear = Linear(tensors[self.name], tensors.get("bias"))

    def projections(self) -> list:
        return [self.linear]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x) -> torch.Tensor:
        """Float32 logits ``[rows, vocab]``: in ``ctx.logits_out`` where the step gave one and the
        product could write there, else in scratch memory."""
        into = ctx.logits_out if ctx.logits_out is not None and ctx.logits_out.shape[0] == x.shape[0] else None
        logits = self.linear(ctx, x, "head.logits", into)
        logits = logits[0] if logits.shape[0] == 1 else logits.sum(dim=0)
        if self.scale != 1.0:
            logits.mul_(self.scale)             # in place: the step's own output tensor stays the one that holds them
        return logits
