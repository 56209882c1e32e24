"""Mixture of experts with group-limited top-k routing and an optional shared expert.

Every expert is a gated feed-forward ``down(f(gate x) * up x)`` without biases.  The router's logits ``W_r x`` are
float32; scores are their softmax over all experts.  Experts form ``groups`` equal groups of neighbours, a group's
score is the largest score in it, and only experts of the ``keep`` best groups can be chosen; each token takes the
``top`` largest of those, weighted by score / (sum of the chosen scores + 1e-20).  A shared expert of its own width
runs for every token and is added unweighted.

Options: ``score="sigmoid"`` (scores are the logits' sigmoids); ``correction`` (a stored number per expert that is added to
the scores for the choice of groups and experts only); ``group_score="top2"`` (a group's score is the sum of its two largest
choice scores); ``renormalize`` off (the weights are the chosen scores as they are); ``activation="clamped"``: an expert is
``down(g' sigmoid(alpha g') (u' + 1))`` with ``g' = min(gate x, limit)`` and ``u' = clamp(up x, -limit, limit)``, the shared expert
with a limit of its own; ``shared_gate``: the shared expert's output is multiplied by ``sigmoid(w_sg . x)``, one number a token,
whose row rides behind the router's rows in one product.

The experts run as ONE gated product over the concatenation of all experts' gate and up rows (the shared expert's
behind them) and ONE down product over the concatenated columns: a token's activations are multiplied by its
routing weight per expert (zero for experts it did not choose) in between, so the down product's sum over its input
IS the weighted sum over experts.  Every matrix is read once per step whatever the routing, which is what a decode
step of more than a few sequences does anyway, and prompts keep the tensor-core tiles full; the price is the
arithmetic of the experts a token did not choose.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import FEED_FORWARDS, Delta, FeedForward, WeightDecl
from .linear import GatedLinear, Linear


@FEED_FORWARDS.register("moe")
class MixtureOfExperts(FeedForward):
    NAMES = {"router": "router.weight", "expert": "experts.{}.", "shared": "shared.", "gate": "gate_proj.weight", "up": "up_proj.weight",
             "down": "down_proj.weight", "correction": "router.correction", "shared_gate": "shared.gate.weight"}

    def __init__(self, hidden: int, experts: int, top: int, inter: int, groups: int = 1, keep: int = 1, shared_inter: int = 0,
                 activation: str = "silu", names: dict | None = None, score: str = "softmax", correction: bool = False,
                 group_score: str = "max", renormalize: bool = True, limit: float = 0.0, shared_limit: float = 0.0, alpha: float = 1.702,
                 shared_gate: bool = False):
        self.hidden, self.experts, self.top, self.inter = int(hidden), int(experts), int(top), int(inter)
        self.groups, self.keep, self.shared_inter = int(groups), int(keep), int(shared_inter or 0)
        if activation != "clamped" and activation not in api.GATE_ACTIVATIONS:
            raise ValueError(f"gate activation {activation!r} is not 'clamped' or one of {sorted(api.GATE_ACTIVATIONS)}")
        if score not in ("softmax", "sigmoid") or group_score not in ("max", "top2"):
            raise ValueError("routing scores are 'softmax' or 'sigmoid', group scores 'max' or 'top2'")
        self.score, self.group_score, self.renormalize = score, group_score, bool(renormalize)
        self.has_correction, self.shared_gate = bool(correction), bool(shared_gate) and bool(shared_inter)
        self.limit, self.shared_limit, self.alpha = float(limit or 0.0), float(shared_limit or 0.0), float(alpha)
        self.correction: torch.Tensor | None = None
        if self.experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{experts} experts do not form {groups} equal groups of which {keep} stay")
        if not 1 <= self.top <= self.keep * (self.experts // self.groups):
            raise ValueError(f"a token cannot choose {top} experts out of {self.keep * (self.experts // self.groups)} allowed ones")
        if self.experts > api.ROUTE_MAX_EXPERTS or self.groups > 32 or self.top > 32:
            raise ValueError(f"the routing kernel takes up to {api.ROUTE_MAX_EXPERTS} experts, 32 groups and 32 choices")
        self.activation = activation
        self.names = {**self.NAMES, **(names or {})}
        self.router: Linear | None = None
        self.gate_up: GatedLinear | None = None
        self.down: Linear | None = None

    def _expert_names(self, prefix: str) -> tuple[str, str, str]:
        n = self.names
        return prefix + n["gate"], prefix + n["up"], prefix + n["down"]

    def _prefixes(self) -> list[tuple[str, int]]:
        out = [(self.names["expert"].format(e), self.inter) for e in range(self.experts)]
        if self.shared_inter:
            out.append((self.names["shared"], self.shared_inter))
        return out

    def weights(self) -> dict[str, WeightDecl]:
        out = {}
        for prefix, inter in self._prefixes():
            gate, up, down = self._expert_names(prefix)
            out[gate] = WeightDecl((inter, self.hidden))
            out[up] = WeightDecl((inter, self.hidden))
            out[down] = WeightDecl((self.hidden, inter))
        out[self.names["router"]] = WeightDecl((self.experts, self.hidden))
        if self.has_correction:
            out[self.names["correction"]] = WeightDecl((self.experts,), init="small")
        if self.shared_gate:
            out[self.names["shared_gate"]] = WeightDecl((1, self.hidden))
        return out

    def bind(self, tensors, dtype, device) -> None:
        names = [self._expert_names(prefix) for prefix, _ in self._prefixes()]
        self.gate_up = GatedLinear(torch.cat([tensors[g] for g, _, _ in names], dim=0), torch.cat([tensors[u] for _, u, _ in names], dim=0),
                                   None, None, "silu" if self.activation == "clamped" else self.activation)
        self.down = Linear(torch.cat([tensors[d] for _, _, d in names], dim=1))
        # the router's sums are float32 in both dtypes; its matrix stays as stored (widening bfloat16 changes nothing)
        router = tensors[self.names["router"]]
        if self.shared_gate:                    # the shared expert's gate row behind the experts' rows
            router = torch.cat([router, tensors[self.names["shared_gate"]].reshape(1, self.hidden).to(router.dtype)], dim=0)
        self.router = Linear(router)
        if self.has_correction:
            self.correction = tensors[self.names["correction"]].to(torch.float32).contiguous()

    def projections(self) -> list:
        return [self.router, self.gate_up.fused, self.down]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x) -> Delta:
        tokens = ctx.n_tokens
        extra = 1 if self.shared_gate else 0
        gates = ctx.scratch("moe.gates", (tokens, self.experts + extra), torch.float32)
        chosen = ctx.scratch("moe.chosen", (tokens, self.top), torch.int32)
        weights = ctx.scratch("moe.weights", (tokens, self.top), torch.float32)
        options = {"score": self.score, "correction": self.correction, "group_score": self.group_score, "renormalize": self.renormalize,
                   "extra": extra}
        if api.route_rows_takes(self.hidden, self.experts + extra):
            api.route_rows(x, self.router.weight, self.top, self.groups, self.keep, gates, chosen, weights, **options)
        else:                                   # rows too wide to stage: the exact product, then the routing
            logits = ctx.scratch("moe.router", (1, tokens, self.experts + extra), torch.float32)
            api.gemm_simt(x, self.router.weight, None, logits)
            api.route_topk(logits, self.top, self.groups, self.keep, gates, chosen, weights, **options)
        if self.activation == "clamped":
            act = ctx.scratch("moe.gate_up.act", (tokens, self.experts * self.inter + self.shared_inter))
            w = self.gate_up.fused.weight
            if api.gemm_tcgen05_usable(x, w) and (tokens > api.SKINNY_TOKENS or api.gemm_tcgen05_splits(tokens, w.shape[0], x.shape[1]) == 1):
                # the clamp and the unit are the gated product's epilogue (the float32 gate and up never reach memory); the
                # routing weights and the shared expert's gate then scale the columns in place
                api.set_label("moe.gate_up")
                api.gemm_tcgen05_clamped(x, w, act, ctx.status, self.limit, self.shared_limit, self.experts * self.inter, self.alpha)
                api.scale_expert_columns(act, self.inter, gates, self.experts, self.shared_inter if self.shared_gate else 0)
            else:                               # the clamp, the unit and the routing weights in one pass over the float32 product
                api.expert_activation(self.gate_up.fused(ctx, x, "moe.gate_up"), act, self.experts, self.inter, self.shared_inter, self.limit,
                                      self.shared_limit, self.alpha, gates, self.shared_gate)
            return self.down.delta(ctx, act, "moe.down")
        act = self.gate_up(ctx, x, "moe.gate_up")
        api.scale_expert_columns(act, self.inter, gates)
        if extra:
            raise NotImplementedError("a gated shared expert goes with the clamped unit")
        return self.down.delta(ctx, act, "moe.down")
