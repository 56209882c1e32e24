"""How a layer's parts are wired around the residual stream.

``pre_norm``: ``h += mixer(norm(h)); h += ffn(norm(h))``, the order of
thinruntime/gpu_runtime.py:10114-10390.  The residual stream is float32; a part's
output is handed on as a :class:`Delta` and added by the next norm's kernel, so the
layer's second addition is done by the following layer's first norm (or by the final
norm).  For long prompts the output projections add their product into the stream themselves
(their tensor-core kernel's epilogue reads and writes the tile once, which spares the
norm kernel a read of the product and a write of the stream); the delta is then empty.

``sandwich``: every sublayer stands between two norms, ``h += norm_after(mixer(norm_before(h)))`` and the same for the
feed-forward, and the layer's end may mix the results of all layers so far into the stream that goes on.  The norm
after a sublayer and the mixing are not kernels of their own: the delta that the sublayer hands on says what is to be
done with it, and the next norm's kernel does it on its way (the layer's last delta reaches the next layer's first
norm, or the final norm).
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import ARRANGEMENTS, Arrangement, Delta, DepthStep


@ARRANGEMENTS.register("pre_norm")
class PreNorm(Arrangement):
    """A layer without a feed-forward leaves out ``ffn_norm`` and ``ffn``: its mixer's output is then what the next
    layer's norm adds.  ``side`` (optional): a side input at the layer's end, which reads the stream with the last
    sublayer's output added and hands on what it adds itself."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "ffn", "side": "side"}
    optional = ("ffn_norm", "ffn", "side")

    def __init__(self, parts):
        super().__init__(parts)
        if ("ffn" in parts) != ("ffn_norm" in parts):
            raise ValueError("a pre-norm layer has a feed-forward and its norm, or neither")

    def mixers(self):
        return [self.parts["mixer"]]

    def device_driven(self) -> bool:
        return all(part.device_driven() for part in self.parts.values())

    def run(self, ctx, residual, pending: Delta | None, caches, states) -> Delta:
        hidden = residual.shape[-1]
        # Between a part's output and the norm that follows nothing else reads the stream, so a part
        # may add its output into it directly instead of handing it on.
        ctx.residual = residual
        normed = ctx.scratch("block.normed", (ctx.n_tokens, hidden))
        self.parts["mixer_norm"].forward(ctx, residual, pending, normed)
        last = self.parts["mixer"].forward(ctx, normed, caches[0], states[0])
        if "ffn" in self.parts:
            self.parts["ffn_norm"].forward(ctx, residual, last, normed)
            last = self.parts["ffn"].forward(ctx, normed)
        if "side" in self.parts:
            last = self.parts["side"].forward(ctx, residual, last)
        return last


@ARRANGEMENTS.register("pre_norm_pair")
class PreNormPair(Arrangement):
    """Two mixers side by side on the same normed input, ``h += left_scale * left(norm(h)) + right_scale *
    right(norm(h))``, then the feed-forward sublayer (if the layer has one).  Each mixer has a cache and states of
    its own.  The weighted sum is formed in float32 from the two output projections' partial sums."""

    roles = {"mixer_norm": "norm", "left": "mixer", "right": "mixer", "ffn_norm": "norm", "ffn": "ffn"}
    optional = ("ffn_norm", "ffn")

    def __init__(self, parts, left_scale: float = 1.0, right_scale: float = 1.0):
        super().__init__(parts)
        if ("ffn" in parts) != ("ffn_norm" in parts):
            raise ValueError("a pre-norm layer has a feed-forward and its norm, or neither")
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)

    def mixers(self):
        return [self.parts["left"], self.parts["right"]]

    def device_driven(self) -> bool:
        return all(part.device_driven() for part in self.parts.values())

    def run(self, ctx, residual, pending: Delta | None, caches, states) -> Delta:
        hidden = residual.shape[-1]
        normed = ctx.scratch("block.normed", (ctx.n_tokens, hidden))
        self.parts["mixer_norm"].forward(ctx, residual, pending, normed)
        ctx.residual = None                 # the branches' outputs are weighted before they reach the stream
        left = self.parts["left"].forward(ctx, normed, caches[0], states[0])
        right = self.parts["right"].forward(ctx, normed, caches[1], states[1])
        both = ctx.scratch("block.pair", (1, ctx.n_tokens, hidden), torch.float32)
        api.weighted_pair(left.tensor, self.left_scale, right.tensor, self.right_scale, both)
        mixed = Delta(both)
        if "ffn" not in self.parts:
            return mixed
        ctx.residual = residual
        self.parts["ffn_norm"].forward(ctx, residual, mixed, normed)
        return self.parts["ffn"].forward(ctx, normed)


@ARRANGEMENTS.register("parallel")
class Parallel(Arrangement):
    """One norm whose output both sublayers read: ``h = norm(x); x += mixer(shift(h)) + ffn(h)``.  ``shift`` (an input
    shift, optional) stands between the norm and the mixer only; the feed-forward (optional) reads ``h`` as it is.  The
    shift's per-sequence state is the arrangement's own."""

    roles = {"norm": "norm", "shift": "shift", "mixer": "mixer", "ffn": "ffn"}
    optional = ("shift", "ffn")

    def mixers(self):
        return [self.parts["mixer"]]

    def state_needs(self):
        return list(self.parts["shift"].state_needs()) if "shift" in self.parts else []

    def device_driven(self) -> bool:
        return all(part.device_driven() for part in self.parts.values())

    def run(self, ctx, residual, pending: Delta | None, caches, states) -> Delta:
        hidden = residual.shape[-1]
        normed = ctx.scratch("block.normed", (ctx.n_tokens, hidden))
        self.parts["norm"].forward(ctx, residual, pending, normed)
        # both sublayers read `normed` and nothing reads the stream before the next norm, so either may add into it
        ctx.residual = residual
        mixer_in = self.parts["shift"].forward(ctx, normed, states[1]) if "shift" in self.parts else normed
        mixed = self.parts["mixer"].forward(ctx, mixer_in, caches[0], states[0])
        if "ffn" not in self.parts:
            return mixed
        fed = self.parts["ffn"].forward(ctx, normed)
        if mixed.tensor is None:
            return fed
        if fed.tensor is None:
            return mixed
        both = ctx.scratch("block.pair", (1, ctx.n_tokens, hidden), torch.float32)
        api.weighted_pair(mixed.tensor, 1.0, fed.tensor, 1.0, both)
        return Delta(both)


@ARRANGEMENTS.register("sandwich")
class Sandwich(Arrangement):
    """``h += post(mixer(pre(h))); h += post'(ffn(pre'(h)))`` with four norms (the feed-forward and its two may be left
    out).  With a ``depth`` part the stream at the layer's end is kept as result ``result_index`` of ``results`` (the
    embedding's output is result 0, kept by the first layer before its first norm) and replaced by the weighted sum of
    results ``0 .. result_index``.  A sublayer's output is normalised before the stream takes it, so no part may add
    into the stream itself."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm", "ffn_norm": "norm", "ffn": "ffn", "ffn_post_norm": "norm",
             "depth": "depth"}
    optional = ("ffn_norm", "ffn", "ffn_post_norm", "depth")

    def __init__(self, parts, result_index: int = 0, results: int = 0):
        super().__init__(parts)
        present = [role in parts for role in ("ffn_norm", "ffn", "ffn_post_norm")]
        if any(present) and not all(present):
            raise ValueError("a sandwich layer has a feed-forward and both of its norms, or none of the three")
        self.result_index, self.results = int(result_index), int(results)
        if "depth" in parts and not 1 <= self.result_index < self.results:
            raise ValueError(f"a layer that mixes results needs its place among them, got {result_index} of {results}")

    def mixers(self):
        return [self.parts["mixer"]]

    def device_driven(self) -> bool:
        return all(part.device_driven() for part in self.parts.values())

    def run(self, ctx, residual, pending: Delta | None, caches, states) -> Delta:
        hidden = residual.shape[-1]
        ctx.residual = None                     # outputs pass a norm before the stream takes them
        depth = self.parts.get("depth")
        kept = None
        if depth is not None:
            kept = ctx.scratch("model.results", (self.results, ctx.n_tokens, hidden), torch.float32)
            if pending is None:                 # the first layer: the embedding's output is result 0
                pending = Delta(None, depth=DepthStep(kept, 0, None))
        normed = ctx.scratch("block.normed", (ctx.n_tokens, hidden))
        self.parts["mixer_norm"].forward(ctx, residual, pending, normed)
        last = self.parts["mixer"].forward(ctx, normed, caches[0], states[0])
        last = Delta(last.tensor, post=self.parts["mixer_post_norm"].after())
        if "ffn" in self.parts:
            self.parts["ffn_norm"].forward(ctx, residual, last, normed)
            last = self.parts["ffn"].forward(ctx, normed)
            last = Delta(last.tensor, post=self.parts["ffn_post_norm"].after())
        if depth is not None:
            last.depth = DepthStep(kept, self.result_index, depth.weight)
        return last
