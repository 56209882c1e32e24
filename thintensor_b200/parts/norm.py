"""RMSNorm and layer norm over the hidden dimension, fused with the residual addition before them.

``y = x * rsqrt(mean(x^2) + eps) * (w + weight_offset)`` with the statistics in float32
(thinruntime/gpu_runtime.py:13028-13039; the fused add form is the reference's
_add_rms_norm_kernel, thinruntime/triton_kernels.py:2580-2614).  ``weight_offset`` is 0
for Llama (thinruntime/model_arch.py:231-233) and 1 for a weight that is stored as its distance from one.

The delta that a norm adds may ask for more on the way (see :class:`~thintensor_b200.parts.base.Delta`): to be
normalised itself before the stream takes it, and for the stream to be replaced, after the addition, by a weighted sum
of the layers' results so far.  The RMS norm's kernel does all of it in its one pass over a row.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import NORMS, Delta, Norm, PostNorm, WeightDecl


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, dim: int, eps: float, weight_offset: float = 0.0, name: str = "weight", init: str | None = None):
        self.dim = int(dim)
        self.eps = float(eps)
        self.weight_offset = float(weight_offset)
        self.name = name                        # what the checkpoint calls the weight, behind the part's prefix
        self.init = init or ("norm" if self.weight_offset == 0.0 else "small")     # how random weights are drawn
        self.weight: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        return {self.name: WeightDecl((self.dim,), init=self.init)}

    def after(self) -> PostNorm:
        """This norm as the one a sublayer's output passes before the stream takes it."""
        return PostNorm(self.weight, self.eps, self.weight_offset)

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name].to(torch.float32).contiguous()

    def vectors(self) -> list[torch.Tensor]:
        return [self.weight]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, residual, delta: Delta | None, out, rows=None) -> None:
        if delta is not None and (delta.post is not None or delta.depth is not None):
            post, depth = delta.post, delta.depth
            if post is not None and delta.tensor is None:
                raise RuntimeError("a delta that is already in the stream cannot be normalised on its way there")
            api.add_rmsnorm_chain(residual, delta.tensor, None if post is None else post.weight, 0.0 if post is None else post.offset,
                                  self.eps if post is None else post.eps, None if depth is None else depth.results,
                                  0 if depth is None else depth.index, None if depth is None else depth.weights, self.weight,
                                  self.weight_offset, self.eps, out, rows)
            return
        api.add_rmsnorm(residual, None if delta is None else delta.tensor, self.weight, self.eps, out, rows, self.weight_offset)   # an empty delta is already in the stream


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """``y = (x - mean(x)) / sqrt(var(x) + eps) * w (+ b)`` with the variance the mean of the squared deviations,
    statistics in float32, fused with the residual addition before it like :class:`RMSNorm`.  ``bias``: whether the
    checkpoint stores one (``bias_name``)."""

    def __init__(self, dim: int, eps: float, bias: bool = False, name: str = "weight", bias_name: str = "bias"):
        self.dim, self.eps, self.bias = int(dim), float(eps), bool(bias)
        self.name, self.bias_name = name, bias_name
        self.weight: torch.Tensor | None = None
        self.shift: torch.Tensor | None = None

    def weights(self) -> dict[str, WeightDecl]:
        out = {self.name: WeightDecl((self.dim,), init="norm")}
        if self.bias:
            out[self.bias_name] = WeightDecl((self.dim,), init="zeros")
        return out

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name].to(torch.float32).contiguous()
        self.shift = tensors[self.bias_name].to(torch.float32).contiguous() if self.bias else None

    def vectors(self) -> list[torch.Tensor]:
        return [self.weight] + ([self.shift] if self.shift is not None else [])

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, residual, delta: Delta | None, out, rows=None) -> None:
        if delta is not None and (delta.post is not None or delta.depth is not None):
            raise NotImplementedError("the layer norm adds plain deltas only")
        api.add_layernorm(residual, None if delta is None else delta.tensor, self.weight, self.shift, self.eps, out, rows)
