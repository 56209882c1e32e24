"""Mixing the layers' results along the depth of the model.

With ``X_0`` the embedding's output and ``X_(i+1)`` the stream at the end of layer ``i`` (before any mixing), the
stream that goes on from layer ``i`` is ``sum(w[j] * X_j for j = 0 .. i + 1)`` with ``i + 2`` learned weights of the
layer.  The part holds the weights; the arrangement hands them, as a
:class:`~thintensor_b200.parts.base.DepthStep`, to the norm kernel that ends the layer, which keeps ``X_(i+1)`` and
forms the sum in float32 while it has the row in registers.
"""
from __future__ import annotations

import torch

from .base import DEPTH_MIXES, Part, WeightDecl


@DEPTH_MIXES.register("weighted_results")
class WeightedResults(Part):
    def __init__(self, count: int, name: str = "weight"):
        self.count = int(count)                 # results mixed: the embedding's output and one per layer up to this one
        self.name = name
        self.weight: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        return {self.name: WeightDecl((self.count,), init="depth")}

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name].to(torch.float32).contiguous()

    def vectors(self) -> list[torch.Tensor]:
        return [self.weight]

    def device_driven(self) -> bool:
        return True
