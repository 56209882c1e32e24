"""Two further attention mixers over the block cache.

``differential_attention``: every query head and every key head carries two maps of ``dim`` numbers (a row is
``[map 1, map 2]``).  Each map is a causal softmax attention of its own over the same values; with a1 and a2 their
outputs, the head's output is ``o = a1 - lam * a2``, divided by ``sqrt(mean(o^2) + eps)`` over the head's ``value_dim``
numbers and multiplied by ``1 - diff``.  ``lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` is one number for the layer,
formed from four learned vectors of ``dim`` numbers in float32 when the weights are bound.  Projections may have
biases.  ``q_gain`` = (coef, every) multiplies the queries at position p by ``1 + coef * ln(floor((p + 1) / every) + 1)``.
A layer with ``own_keys`` off has no key and value projections: its run of the schedule reads an earlier run's cache.
The cache keeps a key head's two maps as one row of ``2 * dim`` numbers.

``pooled_window_attention``: position i sees the keys j with ``0 <= i - j < window`` and, in the same softmax, one mean
key and mean value for every block of ``pool`` tokens that lies wholly before the window (block n, tokens ``n * pool ..
n * pool + pool - 1``, is seen once ``n * pool + pool - 1 <= i - window``); tokens between the last such block and the
window are not seen at all.  Queries and keys are divided by their root mean square per head (no weight); the values are
the keys as projected, before that norm; scores may be capped, ``cap * tanh(s / cap)``.  The means are taken over the
keys and values as the cache holds them and kept in a second, coarser cache (one entry per block), written by the step
that brings a block's last token.  The token cache gives blocks back once neither a window nor an unfinished block needs
them: it keeps the last ``max(window, pool)`` tokens.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .attention import kv_splits
from .base import MIXERS, Delta, KVNeed, Mixer, WeightDecl
from .linear import Linear


def _slice_scratch(ctx, name: str, rows: int, splits: int, per_row: int, maps: int = 1):
    if splits <= 1:
        return None, None
    return (ctx.scratch(name + ".part_acc", (rows * splits * maps * per_row,), torch.float32),
            ctx.scratch(name + ".part_ml", (rows * splits * maps * 2,), torch.float32))


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight", "q_bias": "q_proj.bias",
             "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "lq1": "lambda_q1", "lk1": "lambda_k1", "lq2": "lambda_q2", "lk2": "lambda_k2"}

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, value_dim: int, scale: float, diff: float, eps: float,
                 bias: bool = False, q_gain: tuple | None = None, own_keys: bool = True, names: dict | None = None):
        self.hidden, self.heads, self.kv_heads, self.dim, self.value_dim = int(hidden), int(heads), int(kv_heads), int(dim), int(value_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} key/value heads")
        api.check_head_dim(2 * self.dim)
        api.check_head_dim(self.value_dim)
        self.scale, self.diff, self.eps = float(scale), float(diff), float(eps)
        self.bias, self.own_keys = bool(bias), bool(own_keys)
        self.q_gain = None if q_gain is None else (float(q_gain[0]), int(q_gain[1]))
        self.names = {**self.NAMES, **(names or {})}
        self.lam = 0.0
        self.projection: Linear | None = None       # q (and k, v where the layer has its own)
        self.out: Linear | None = None
        self.no_rotation: torch.Tensor | None = None
        self.on_tensor_cores: bool | None = None

    def weights(self) -> dict[str, WeightDecl]:
        n = self.names
        rows = {"q": self.heads * 2 * self.dim}
        if self.own_keys:
            rows.update({"k": self.kv_heads * 2 * self.dim, "v": self.kv_heads * self.value_dim})
        out = {n[key]: WeightDecl((count, self.hidden)) for key, count in rows.items()}
        if self.bias:
            out.update({n[key + "_bias"]: WeightDecl((count,)) for key, count in rows.items()})
        out.update({n[key]: WeightDecl((self.dim,), init="small") for key in ("lq1", "lk1", "lq2", "lk2")})
        out[n["o"]] = WeightDecl((self.hidden, self.heads * self.value_dim))
        return out

    def cache_need(self) -> KVNeed:
        return KVNeed(self.kv_heads, 2 * self.dim, None, None if self.value_dim == 2 * self.dim else self.value_dim)

    @property
    def pair_dims(self) -> tuple[int, int]:
        """What a (query, key) pair costs: two scores of ``dim`` numbers and the value taken twice, once per map."""
        return 2 * self.dim, 2 * self.value_dim

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        keys = ("q", "k", "v") if self.own_keys else ("q",)
        weight = torch.cat([tensors[n[key]] for key in keys], dim=0)
        bias = torch.cat([tensors[n[key + "_bias"]].float() for key in keys]) if self.bias else None
        self.projection = Linear(weight, bias)
        self.out = Linear(tensors[n["o"]])
        f = {key: tensors[n[key]].to(torch.float32) for key in ("lq1", "lk1", "lq2", "lk2")}
        lam = torch.exp((f["lq1"] * f["lk1"]).sum()) - torch.exp((f["lq2"] * f["lk2"]).sum()) + torch.tensor(self.diff, dtype=torch.float32)
        self.lam = float(lam)
        self.no_rotation = torch.zeros(1, dtype=torch.float32, device=device)

    def projections(self) -> list:
        return [self.projection, self.out]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x, cache, states) -> Delta:
        if cache is None or cache.k_pool is None:
            raise RuntimeError("attention needs a cache with storage")
        if cache.writes != self.own_keys:
            raise RuntimeError("a differential layer writes the cache exactly when it projects keys and values of its own")
        table = ctx.tables[cache.group]
        row = 2 * self.dim
        projected = self.projection(ctx, x, "attention.qkv")
        q = ctx.scratch("attention.q", (ctx.n_tokens, self.heads * row))
        api.qk_norm_rope_append(projected, None, None, 0.0, self.no_rotation, 0, False, 1.0, q, cache.k_pool if cache.writes else None,
                                cache.v_pool if cache.writes else None, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens,
                                self.heads, self.kv_heads, row, self.value_dim, ctx.status, q_gain=self.q_gain)
        mixed = ctx.scratch("attention.mixed", (ctx.n_tokens, self.heads * self.value_dim))
        if self.on_tensor_cores is None:        # asked once: the answer depends on the sizes and the activations' type only
            self.on_tensor_cores = api.attention_forms_on_tensor_cores(q.dtype, True, self.heads, self.kv_heads, self.dim, self.value_dim)
        if self.on_tensor_cores:
            splits = kv_splits(ctx, ctx.n_tokens * self.kv_heads, 128, 3 * api.sm_count(q.device))
        else:
            splits = kv_splits(ctx, ctx.n_tokens * self.heads, 256, 8 * api.sm_count(q.device))
        part_acc, part_ml = _slice_scratch(ctx, "differential", ctx.n_tokens * self.heads, splits, self.value_dim, maps=2)
        api.differential_attention(q, cache.k_pool, cache.v_pool, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads,
                                   self.kv_heads, self.dim, self.value_dim, self.scale, self.lam, 1.0 - self.diff, self.eps, splits, mixed,
                                   part_acc, part_ml, ctx.status)
        return self.out.delta(ctx, mixed, "attention.out")


@MIXERS.register("pooled_window_attention")
class PooledWindowAttention(Mixer):
    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "o": "o_proj.weight"}

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, scale: float, eps: float, window: int, pool: int,
                 softcap: float | None = None, names: dict | None = None):
        self.hidden, self.heads, self.kv_heads, self.dim = int(hidden), int(heads), int(kv_heads), int(dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} key/value heads")
        api.check_head_dim(self.dim)
        self.scale, self.eps = float(scale), float(eps)
        self.window, self.pool = int(window), int(pool)
        if self.window < 1 or self.pool < 1:
            raise ValueError("the window and the blocks hold at least one token")
        self.softcap = 0.0 if not softcap else float(softcap)
        self.names = {**self.NAMES, **(names or {})}
        self.projection: Linear | None = None       # q, then k
        self.out: Linear | None = None
        self.no_rotation: torch.Tensor | None = None
        self.on_tensor_cores: bool | None = None

    def weights(self) -> dict[str, WeightDecl]:
        n = self.names
        return {n["q"]: WeightDecl((self.heads * self.dim, self.hidden)), n["k"]: WeightDecl((self.kv_heads * self.dim, self.hidden)),
                n["o"]: WeightDecl((self.hidden, self.heads * self.dim))}

    def cache_need(self) -> KVNeed:
        return KVNeed(self.kv_heads, self.dim, max(self.window, self.pool))

    def summary_need(self) -> KVNeed:
        return KVNeed(self.kv_heads, self.dim, None, None, self.pool)

    def visible_pairs(self, tokens: int) -> float:
        """(query, key) pairs of one sequence of ``tokens`` tokens: the window's tokens and the whole blocks before it."""
        return float(sum(min(i + 1, self.window) + max(0, i - self.window + 1) // self.pool for i in range(tokens)))

    def bind(self, tensors, dtype, device) -> None:
        n = self.names
        self.projection = Linear(torch.cat([tensors[n["q"]], tensors[n["k"]]], dim=0))
        self.out = Linear(tensors[n["o"]])
        self.no_rotation = torch.zeros(1, dtype=torch.float32, device=device)

    def projections(self) -> list:
        return [self.projection, self.out]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x, cache, states) -> Delta:
        if cache is None or cache.k_pool is None or cache.summary is None or cache.summary.k_pool is None:
            raise RuntimeError("window attention with pooled blocks needs a cache and a coarser cache with storage")
        if not cache.writes:
            raise RuntimeError("window attention with pooled blocks keeps a cache of its own")
        coarse = cache.summary
        table, mean_table = ctx.tables[cache.group], ctx.tables[coarse.group]
        projected = self.projection(ctx, x, "attention.qkv")
        q = ctx.scratch("attention.q", (ctx.n_tokens, self.heads * self.dim))
        api.qk_norm_rope_append(projected, None, None, self.eps, self.no_rotation, 0, False, 1.0, q, cache.k_pool, cache.v_pool, table,
                                ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads, self.kv_heads, self.dim, self.dim,
                                ctx.status, unit_norm=True, value_from_keys=True)
        # the blocks whose last token this step brings: at most one more than the step's longest share holds whole blocks
        api.pool_blocks(cache.k_pool, cache.v_pool, table, coarse.k_pool, coarse.v_pool, mean_table, ctx.cu, ctx.len_before, ctx.sequences,
                        ctx.max_new // self.pool + 1, self.kv_heads, self.dim, self.dim, self.pool, ctx.status)
        mixed = ctx.scratch("attention.mixed", (ctx.n_tokens, self.heads * self.dim))
        splits = 1
        if ctx.decode:      # the keys a position sees: its window and the blocks before it
            most = self.window + ctx.max_total // self.pool
            if self.on_tensor_cores is None:        # asked once: the answer depends on the sizes and the activations' type only
                self.on_tensor_cores = api.attention_forms_on_tensor_cores(q.dtype, False, self.heads, self.kv_heads, self.dim, self.dim)
            if self.on_tensor_cores:
                splits = max(1, min(3 * api.sm_count(q.device) // max(ctx.n_tokens * self.kv_heads, 1), most // 128, 64))
            else:
                splits = max(1, min(8 * api.sm_count(q.device) // max(ctx.n_tokens * self.heads, 1), most // 256, 64))
        part_acc, part_ml = _slice_scratch(ctx, "window", ctx.n_tokens * self.heads, splits, self.dim)
        api.pooled_window_attention(q, cache.k_pool, cache.v_pool, table, coarse.k_pool, coarse.v_pool, mean_table, self.pool, ctx.cu,
                                    ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads, self.kv_heads, self.dim, self.scale,
                                    self.softcap, self.window, splits, mixed, part_acc, part_ml, ctx.status)
        return self.out.delta(ctx, mixed, "attention.out")
