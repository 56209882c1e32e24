"""Dense feed-forwards.  Gated: ``down(f(gate(x)) * up(x))``, f = ``silu(g) = g / (1 + exp(-g))`` by default
(thinruntime/gpu_runtime.py:10286-10366; the activation at :10351 and
thinruntime/triton_kernels.py:2760-2774), or ``relu`` or ``gelu_tanh`` (``activation``).  ``names`` gives the
checkpoint's names of the gate, up and down matrices behind the part's prefix.

Ungated (``mlp``): ``down(f(up(x)))`` with f one of the gate activations or ``xielu``, which has two learned numbers
(p, q) per layer: ``softplus(p) z^2 + z / 2`` for z > 0 and ``(1 / 2 + softplus(q)) (exp(z) - 1 - z) + z / 2`` otherwise."""
from __future__ import annotations

import torch

from ..kernels import api
from .base import FEED_FORWARDS, Delta, FeedForward, WeightDecl
from .linear import GatedLinear, Linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    def __init__(self, hidden: int, inter: int, bias: bool = False, activation: str = "silu", names: dict | None = None):
        self.hidden, self.inter, self.bias = int(hidden), int(inter), bool(bias)
        if activation not in api.GATE_ACTIVATIONS:
            raise ValueError(f"gate activation {activation!r} is not one of {sorted(api.GATE_ACTIVATIONS)}")
        self.activation = activation
        self.names = {**self.NAMES, **(names or {})}
        self.gate_up: GatedLinear | None = None
        self.down: Linear | None = None

    def weights(self) -> dict[str, WeightDecl]:
        n = self.names
        out = {
            n["gate"]: WeightDecl((self.inter, self.hidden)),
            n["up"]: WeightDecl((self.inter, self.hidden)),
            n["down"]: WeightDecl((self.hidden, self.inter)),
        }
        if self.bias:
            out.update({"gate_proj.bias": WeightDecl((self.inter,)), "up_proj.bias": WeightDecl((self.inter,)),
                        "down_proj.bias": WeightDecl((self.hidden,))})
        return out

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        self.gate_up = GatedLinear(tensors[n["gate"]], tensors[n["up"]],
                                   tensors.get("gate_proj.bias"), tensors.get("up_proj.bias"), self.activation)
        self.down = Linear(tensors[n["down"]], tensors.get("down_proj.bias"))

    def projections(self) -> list:
        return [self.gate_up.fused, self.down]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x) -> Delta:
        act = self.gate_up(ctx, x, "ffn.gate_up")
        return self.down.delta(ctx, act, "ffn.down")


@FEED_FORWARDS.register("mlp")
class Mlp(FeedForward):
    NAMES = {"up": "up_proj.weight", "down": "down_proj.weight", "act": "act"}

    def __init__(self, hidden: int, inter: int, activation: str = "gelu_tanh", names: dict | None = None):
        self.hidden, self.inter = int(hidden), int(inter)
        if activation not in api.UNARY_ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(api.UNARY_ACTIVATIONS)}")
        self.activation = activation
        self.names = {**self.NAMES, **(names or {})}
        self.up: Linear | None = None
        self.down: Linear | None = None
        self.act_params = (0.0, 0.0)            # xielu: (softplus(p), 1 / 2 + softplus(q)), float32 arithmetic

    def weights(self) -> dict[str, WeightDecl]:
        n = self.names
        out = {n["up"]: WeightDecl((self.inter, self.hidden)), n["down"]: WeightDecl((self.hidden, self.inter))}
        if self.activation == "xielu":
            out[n["act"]] = WeightDecl((2,), init="small")
        return out

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        self.up = Linear(tensors[n["up"]])
        self.down = Linear(tensors[n["down"]])
        if self.activation == "xielu":
            pq = torch.nn.functional.softplus(tensors[n["act"]].to(torch.float32)).cpu()
            self.act_params = (float(pq[0]), float(torch.tensor(0.5, dtype=torch.float32) + pq[1]))

    def projections(self) -> list:
        return [self.up, self.down]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x) -> Delta:
        act = ctx.scratch("ffn.up.act", (x.shape[0], self.inter))
        api.activation(self.up(ctx, x, "ffn.up"), act, self.activation, *self.act_params)
        return self.down.delta(ctx, act, "ffn.down")
