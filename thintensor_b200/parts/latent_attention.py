"""Causal softmax attention whose keys and values are expansions of one cached latent per token.

Queries take a low-rank path: ``c_q = rmsnorm(W_dq x)`` (weight and eps), ``q = W_uq c_q``, per head ``dim``
unrotated numbers followed by ``rot_dim`` numbers that are rotated by the position.  Keys and values share a
latent: ``W_dkv x`` has ``kv_rank + rot_dim`` rows; the first ``kv_rank``, RMS-normed, are the latent ``c``, the
rest are one rotated key part that all heads share.  Per head ``k = [W_uk c | k_rot]`` and ``v = W_uv c``; the
score is ``(q . k) * scale`` over the last ``window`` positions (or all of them), softmax, then ``W_o`` on the
concatenated heads.

Options: no low-rank query path at all (``q_rank`` None: ``q = W_q x``, tensor ``q``); a rotation that pairs neighbouring
numbers and multiplies cosines and sines by a constant (the position encoding's ``interleaved`` and
``attention_scaling``); every head's output multiplied by ``sigmoid(W_g x)_h``, one number per head (``gate="head"``).  Where
the queries are projected directly, ONE product makes ``[kv latent | shared key part | queries | gate]``.

Only ``[c | k_rot]`` is cached: one row per token, one key/value head, no value pool.  Decoding (and every step
the tensor-core kernels do not take) never forms keys or values: the kernel folds ``W_uk`` into the query
(``a = W_uk_h^T q_h``, so that ``q_h . W_uk_h c = a . c``) and applies ``W_uv_h`` once to the softmax-weighted sum of
latents.  Prompts in bfloat16 whose heads have a size the tcgen05 attention kernel takes (``dim + rot_dim ==
value_dim`` of 64 or 128) expand the latents the step can see into per-head keys and values for the length of the
step, in scratch memory laid out like blocks of the ordinary cache, with one product over ``[W_uk; W_uv]``, and run
that kernel on them: a prompt's arithmetic is then that of ordinary heads (``dim + rot_dim + value_dim`` numbers a
pair instead of ``2 kv_rank + rot_dim``) and runs on the tensor cores.  Norms, positions, angles, scores and softmax
weights are float32 in both dtypes.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .attention import kv_splits
from .base import MIXERS, POSITION_ENCODINGS, Delta, KVNeed, Mixer, RotaryTable, WeightDecl
from .linear import Linear
from .spec import PartSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    NAMES = {"dq": "q_a_proj.weight", "dq_norm": "q_a_norm.weight", "uq": "q_b_proj.weight", "dkv": "kv_a_proj.weight",
             "dkv_norm": "kv_a_norm.weight", "uk": "k_b_proj.weight", "uv": "v_b_proj.weight", "o": "o_proj.weight",
             "q": "q_proj.weight", "g": "g_proj.weight"}

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, value_dim: int, q_rank: int | None, kv_rank: int, scale: float,
                 eps: float, position: PartSpec | None = None, window: int | None = None, names: dict | None = None,
                 gate: str | None = None):
        self.hidden, self.heads, self.dim, self.rot_dim = int(hidden), int(heads), int(dim), int(rot_dim)
        self.value_dim, self.q_rank, self.kv_rank = int(value_dim), int(q_rank or 0), int(kv_rank)
        if gate not in (None, "head"):
            raise ValueError(f"latent attention gates its heads ('head') or nothing, not {gate!r}")
        self.gate = gate
        self.scale, self.eps = float(scale), float(eps)
        self.window = None if not window else int(window)
        if self.kv_rank > api.LATENT_MAX_RANK or self.kv_rank + self.rot_dim > api.LATENT_MAX_ROW or self.dim > api.LATENT_MAX_DIM:
            raise ValueError(f"latent attention takes latents of up to {api.LATENT_MAX_RANK} numbers, cache rows of up to "
                             f"{api.LATENT_MAX_ROW} and {api.LATENT_MAX_DIM} unrotated numbers per head")
        self.names = {**self.NAMES, **(names or {})}
        position = position or PartSpec("none", {"head_dim": max(self.rot_dim, 1)})
        self.position = POSITION_ENCODINGS.build(position.kind, dict(position.params))
        if self.position.kind not in ("rotary", "none"):
            raise ValueError(f"latent attention applies rotary position encodings or none, not one of kind {self.position.kind!r}")
        self.rot: RotaryTable | None = None
        self.down: Linear | None = None
        self.up_q: Linear | None = None
        self.out: Linear | None = None

    def weights(self) -> dict[str, WeightDecl]:
        n = self.names
        if self.q_rank:
            queries = {n["dq"]: WeightDecl((self.q_rank, self.hidden)), n["dq_norm"]: WeightDecl((self.q_rank,), init="norm"),
                       n["uq"]: WeightDecl((self.heads * (self.dim + self.rot_dim), self.q_rank))}
        else:
            queries = {n["q"]: WeightDecl((self.heads * (self.dim + self.rot_dim), self.hidden))}
        gate = {n["g"]: WeightDecl((self.heads, self.hidden))} if self.gate else {}
        return {
            **queries,
            n["dkv"]: WeightDecl((self.kv_rank + self.rot_dim, self.hidden)),
            n["dkv_norm"]: WeightDecl((self.kv_rank,), init="norm"),
            n["uk"]: WeightDecl((self.heads * self.dim, self.kv_rank)),
            n["uv"]: WeightDecl((self.heads * self.value_dim, self.kv_rank)),
            **gate,
            n["o"]: WeightDecl((self.hidden, self.heads * self.value_dim)),
        }

    @property
    def pair_dims(self) -> tuple[int, int]:
        """Numbers of a head's score product and of its value, for the benchmarks' FLOP model."""
        return self.dim + self.rot_dim, self.value_dim

    def cache_need(self) -> KVNeed:
        return KVNeed(1, self.kv_rank + self.rot_dim, self.window, 0)       # one row per token, values read from the key rows

    def bind(self, tensors, dtype, device) -> None:
        self.position.bind({}, dtype, device)
        if self.position.kind == "rotary":
            self.rot = self.position.rotary()
            if self.rot.rotary_dim % 2 or self.rot.rotary_dim > self.rot_dim:
                raise ValueError(f"the rotation takes an even number of at most {self.rot_dim} numbers, got {self.rot.rotary_dim}")
        else:
            self.rot = RotaryTable(torch.zeros(1, dtype=torch.float32, device=device), 0, 1.0)
        n = self.names
        if self.q_rank:
            rows = [tensors[n["dq"]], tensors[n["dkv"]]]                    # [q latent | kv latent | shared key part]
            self.up_q = Linear(tensors[n["uq"]])
            self.q_norm = tensors[n["dq_norm"]].to(torch.float32).contiguous()
        else:
            rows = [tensors[n["dkv"]], tensors[n["q"]]]                     # [kv latent | shared key part | queries]
            self.up_q, self.q_norm = None, None
        if self.gate:
            rows.append(tensors[n["g"]])                                    # one gate number per head behind everything else
        self.down = Linear(torch.cat(rows, dim=0))
        self.out = Linear(tensors[n["o"]])
        self.kv_norm = tensors[n["dkv_norm"]].to(torch.float32).contiguous()
        self.w_key, self.w_value = tensors[n["uk"]].contiguous(), tensors[n["uv"]].contiguous()
        self.expander = Linear(torch.cat([self.w_key, self.w_value], dim=0))        # [W_uk; W_uv]: a latent into all heads' keys and values

    def projections(self) -> list:
        return [p for p in (self.down, self.up_q, self.expander, self.out) if p is not None]

    def vectors(self) -> list[torch.Tensor]:
        return [v for v in (self.q_norm, self.kv_norm) if v is not None]

    def device_driven(self) -> bool:
        return True

    def forward(self, ctx, x, cache, states) -> Delta:
        if cache is None or cache.k_pool is None:
            raise RuntimeError("latent attention needs a cache with storage")
        table = ctx.tables[cache.group]
        rot = self.rot
        down = self.down(ctx, x, "latent.down")
        front = self.q_rank + self.kv_rank + self.rot_dim
        head_gate = down[:, :, down.shape[2] - self.heads:] if self.gate else None
        q_latent = ctx.scratch("latent.q_latent", (ctx.n_tokens, self.q_rank)) if self.q_rank else None
        api.latent_prepare(down[:, :, :front], self.q_rank, self.kv_rank, self.rot_dim, self.q_norm, self.kv_norm, self.eps, rot.inv_freq,
                           rot.rotary_dim, q_latent, cache.k_pool if cache.writes else None, table, ctx.cu, ctx.len_before,
                           ctx.sequences, ctx.n_tokens, ctx.status, interleaved=rot.interleaved, rot_scale=rot.attention_scaling)
        if self.q_rank:
            q = self.up_q(ctx, q_latent, "latent.up_q")
        else:
            q = down[:, :, front:front + self.heads * (self.dim + self.rot_dim)]
        mixed = ctx.scratch("latent.mixed", (ctx.n_tokens, self.heads * self.value_dim))
        if self.expands(ctx, x):
            self.attend_expanded(ctx, q, cache, table, mixed)
            if head_gate is not None:
                api.sigmoid_gate(mixed, head_gate, self.value_dim)
            return self.out.delta(ctx, mixed, "latent.out")
        splits, tensor_cores = 1, False
        reach = ctx.max_total if self.window is None else min(self.window, ctx.max_total)
        if (ctx.decode and api.latent_decode_tensor_cores(mixed.dtype, self.kv_rank, self.rot_dim)
                and -(-reach // api.LATENT_DECODE_SLICE) <= 256):
            # decoding on the tensor cores: the heads of a token are the rows of both products, the keys go in slices of 64
            splits, tensor_cores = -(-reach // api.LATENT_DECODE_SLICE), True
        elif ctx.decode:
            # keys of a decode step are cut into slices until the (token, head) warps fill the GPU; a window bounds the keys
            splits = min(kv_splits(ctx, ctx.n_tokens * self.heads, 64, 16 * api.sm_count(ctx.status.device)), max(1, reach // 64))
        absorbed = ctx.scratch("latent.absorbed", (ctx.n_tokens * self.heads * (self.kv_rank + self.rot_dim),), torch.float32)
        part_acc = ctx.scratch("latent.part_acc", (ctx.n_tokens * self.heads * splits * self.kv_rank,), torch.float32)
        part_ml = ctx.scratch("latent.part_ml", (ctx.n_tokens * self.heads * splits * 2,), torch.float32)
        api.latent_attention(q, self.w_key, self.w_value, cache.k_pool, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens,
                             self.heads, self.dim, self.rot_dim, self.value_dim, self.kv_rank, rot.inv_freq, rot.rotary_dim, self.scale,
                             self.window or 0, splits, mixed, absorbed, part_acc, part_ml, ctx.status, tensor_cores,
                             interleaved=rot.interleaved, rot_scale=rot.attention_scaling, head_gate=head_gate)
        return self.out.delta(ctx, mixed, "latent.out")

    # ------------------------------------------------------------ prompts on the tensor cores
    EXPAND_FROM = 128           # packed tokens from which a step of prompts is expanded

    def expands(self, ctx, x) -> bool:
        head = self.dim + self.rot_dim
        return (not ctx.decode and ctx.n_tokens >= self.EXPAND_FROM and x.dtype == torch.bfloat16 and head == self.value_dim
                and self.w_key.dtype == torch.bfloat16 and api.attention_tcgen05_supports(x.dtype, self.heads, self.heads, head))

    def expansion_bound(self, ctx, width: int) -> int:
        """Temporary blocks the step can need, from the step's shape alone (a replayed step has other lengths): every
        sequence sees its new tokens and at most ``window - 1`` before them, in blocks of 64 that may be cut at both ends."""
        if self.window is None:
            return ctx.sequences * width
        return min(ctx.sequences * width, (ctx.n_tokens + ctx.sequences * (self.window - 1)) // 64 + 2 * ctx.sequences)

    def attend_expanded(self, ctx, q, cache, table, mixed) -> None:
        head = self.dim + self.rot_dim
        blocks = self.expansion_bound(ctx, table.shape[1])
        plan = ctx.scratch("latent.plan", (2 * ctx.sequences + 1,), torch.int32)
        table_tmp = ctx.scratch("latent.table", tuple(table.shape), torch.int32)
        latents = ctx.scratch("latent.visible", (blocks * 64, self.kv_rank))
        keys = ctx.scratch("latent.keys", (blocks, self.heads, 64, head))
        values = ctx.scratch("latent.values", (blocks, self.heads, self.value_dim, 64))
        api.latent_expand(cache.k_pool, table, ctx.cu, ctx.len_before, ctx.sequences, self.window or 0, blocks, self.heads, self.dim,
                          self.rot_dim, self.kv_rank, plan, table_tmp, latents, keys, ctx.status)
        expanded = self.expander(ctx, latents, "latent.expand")
        api.latent_scatter(expanded, self.heads, self.dim, self.rot_dim, self.value_dim, keys, values)
        queries = ctx.scratch("latent.queries", (ctx.n_tokens, self.heads * head))
        api.latent_queries(q, self.heads, self.dim, self.rot_dim, self.rot.inv_freq, self.rot.rotary_dim, ctx.cu, ctx.len_before,
                           ctx.sequences, ctx.n_tokens, queries, interleaved=self.rot.interleaved, rot_scale=self.rot.attention_scaling)
        api.attention_tcgen05(queries, keys, values, table_tmp, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads, self.heads,
                              head, self.scale, self.window or 0, mixed, ctx.status)
