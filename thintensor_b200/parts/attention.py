"""Causal grouped-query attention over the block cache.

For each token: q, k, v projections of the normed hidden state (one fused matrix),
position encoding on q and k, k and v appended to the sequence's cache, softmax
attention of q over every cached key of its sequence (or the last ``window`` of them)
with query head h reading key/value head ``h // (heads / kv_heads)`` and scores scaled
by ``head_dim ** -0.5`` (or ``scale``), then the output projection
(thinruntime/gpu_runtime.py:10151-10249 and 8913-8961).

Options beyond that form, each a parameter: value heads of another size than key heads
(``value_dim``); queries and keys divided by their root mean square per head and multiplied
by a weight of ``head_dim`` numbers that all heads share, before the rotation
(``qk_norm_eps``); a learned number per query head whose exponential joins the softmax
denominator without a key or a value (``sink``); a rotation that pairs neighbouring numbers
(the position encoding's ``interleaved``); a short causal convolution over time on every channel
of q, k and v right after their projections, ``y_t = sum_j w[:, j] u_(t - taps + 1 + j)`` with zeros before the
sequence (``conv`` taps; the last ``taps - 1`` projected rows are a per-sequence state); scores capped by
``softcap * tanh(s / softcap)``; a bias that grows with the distance, ``slope_h * (i - j)`` taken off the score with
``slope_h = 2 ** (-slope_exponent * (h + 1) / heads)``; the concatenated heads multiplied by ``sigmoid(W_g x)`` before the
output projection (``gate="elementwise"``, or ``"head"`` for one number per head); no key and value projections at
all, for a run of the schedule that reads an earlier run's cache (``own_keys`` off); a cache that keeps more tokens than
the layer's own window (``cache_window``, for the readers of its cache; -1: every token).  A layer that uses any of them runs the general
kernels: one that normalises, rotates and appends, and the exact attention.
"""
from __future__ import annotations

import torch

from ..kernels import api
from .base import MIXERS, POSITION_ENCODINGS, Delta, KVNeed, Mixer, RotaryTable, StateNeed, WeightDecl
from .linear import Linear
from .spec import PartSpec


def kv_splits(ctx, parallel_units: int, keys_per_slice: int, target_units: int) -> int:
    """Into how many slices the keys of a decode step are cut so that the grid fills the
    GPU: ``parallel_units`` is how many independent units (warps or CTAs) the step has
    without slicing, ``target_units`` how many the GPU wants.  Depends only on the step's
    shape and the length bound, never on the lengths on the device."""
    if not ctx.decode:
        return 1
    want = target_units // max(parallel_units, 1)
    most = ctx.max_total // keys_per_slice
    return max(1, min(want, most, 64))


@MIXERS.register("attention")
class CausalAttention(Mixer):
    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sink": "sinks", "g": "g_proj.weight",
             "q_conv": "q_conv.weight", "k_conv": "k_conv.weight", "v_conv": "v_conv.weight"}

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, position: PartSpec | None = None,
                 bias: bool = False, window: int | None = None, scale: float | None = None, value_dim: int | None = None,
                 qk_norm_eps: float | None = None, sink: bool = False, names: dict | None = None, conv: int | None = None,
                 softcap: float | None = None, slope_exponent: float | None = None, gate: str | None = None, own_keys: bool = True,
                 cache_window: int | None = None):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} key/value heads")
        api.check_head_dim(self.head_dim)
        self.value_dim = self.head_dim if value_dim is None else int(value_dim)
        api.check_head_dim(self.value_dim)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.sink = bool(sink)
        self.names = {**self.NAMES, **(names or {})}
        self.q_norm: torch.Tensor | None = None
        self.k_norm: torch.Tensor | None = None
        self.sinks: torch.Tensor | None = None
        self.bias = bool(bias)
        self.conv = int(conv) if conv else 0
        if self.conv and not 1 <= self.conv <= 8:
            raise ValueError("the convolution kernel takes 1 to 8 taps")
        self.softcap = float(softcap) if softcap else 0.0
        self.slope_exponent = None if slope_exponent is None else float(slope_exponent)
        if gate not in (None, "elementwise", "head"):
            raise ValueError(f"an output gate is 'elementwise' or 'head', not {gate!r}")
        self.gate = gate
        self.own_keys = bool(own_keys)
        self.cache_window = None if not cache_window else int(cache_window)       # -1: the cache keeps every token
        self.slopes: torch.Tensor | None = None
        self.conv_weight: torch.Tensor | None = None
        self.window = None if not window else int(window)
        self.scale = float(scale) if scale is not None else self.head_dim ** -0.5
        position = position or PartSpec("none", {"head_dim": self.head_dim})
        self.position = POSITION_ENCODINGS.build(position.kind, dict(position.params))
        if self.position.kind not in ("rotary", "none"):
            raise ValueError(f"attention applies rotary position encodings or none, not one of kind {self.position.kind!r}")
        self.rot: RotaryTable | None = None         # what the kernels rotate by; rotary_dim 0 switches rotation off
        self.qkv: Linear | None = None
        self.q_only: Linear | None = None
        self.out: Linear | None = None

    # -------------------------------------------------------------- declarations
    def weights(self) -> dict[str, WeightDecl]:
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        n = self.names
        out = {n["q"]: WeightDecl((q, self.hidden))}
        if self.own_keys:
            out[n["k"]] = WeightDecl((kv, self.hidden))
            out[n["v"]] = WeightDecl((self.kv_heads * self.value_dim, self.hidden))
        out[n["o"]] = WeightDecl((self.hidden, self.heads * self.value_dim))
        if self.qk_norm_eps is not None:
            out[n["q_norm"]] = WeightDecl((self.head_dim,), init="norm")
            if self.own_keys:
                out[n["k_norm"]] = WeightDecl((self.head_dim,), init="norm")
        if self.conv:
            out[n["q_conv"]] = WeightDecl((q, self.conv), init="small")
            if self.own_keys:
                out[n["k_conv"]] = WeightDecl((kv, self.conv), init="small")
                out[n["v_conv"]] = WeightDecl((self.kv_heads * self.value_dim, self.conv), init="small")
        if self.gate:
            out[n["g"]] = WeightDecl((self.gate_cols, self.hidden))
        if self.sink:
            out[n["sink"]] = WeightDecl((self.heads,))
        if self.bias:
            out.update({
                "q_proj.bias": WeightDecl((q,)), "k_proj.bias": WeightDecl((kv,)), "v_proj.bias": WeightDecl((kv,)),
                "o_proj.bias": WeightDecl((self.hidden,)),
            })
        return out

    @property
    def gate_cols(self) -> int:
        return 0 if not self.gate else (self.heads if self.gate == "head" else self.heads * self.value_dim)

    @property
    def conv_channels(self) -> int:
        """What passes the convolution: q, and k and v where the layer projects them."""
        return self.heads * self.head_dim + (self.kv_heads * (self.head_dim + self.value_dim) if self.own_keys else 0)

    def cache_need(self) -> KVNeed:
        window = self.window
        if window is not None and self.cache_window:
            window = None if self.cache_window < 0 else max(window, self.cache_window)
        return KVNeed(self.kv_heads, self.head_dim, window, None if self.value_dim == self.head_dim else self.value_dim)

    def state_needs(self) -> list[StateNeed]:
        return [StateNeed((self.conv - 1, self.conv_channels), torch.float32)] if self.conv > 1 else []

    @property
    def general(self) -> bool:
        """Whether the layer needs the general kernels (see the module's text)."""
        return (self.value_dim != self.head_dim or self.qk_norm_eps is not None or self.sink or bool(self.conv) or self.softcap > 0.0
                or self.slope_exponent is not None or self.gate is not None or not self.own_keys
                or (self.rot is not None and self.rot.interleaved and self.rot.rotary_dim > 0))

    def bind(self, tensors, dtype, device) -> None:
        self.position.bind({}, dtype, device)
        if self.position.kind == "rotary":
            self.rot = self.position.rotary()
            if self.rot.rotary_dim % 2 or not 0 <= self.rot.rotary_dim <= self.head_dim:
                raise ValueError(f"the rotary part must be even and at most the head size {self.head_dim}, got {self.rot.rotary_dim}")
        else:
            self.rot = RotaryTable(torch.zeros(1, dtype=torch.float32, device=device), 0, 1.0)
        n = self.names
        if self.general and self.bias:
            raise ValueError("attention with a value size of its own, a query/key norm, a sink or an interleaved rotation takes no biases")
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm = tensors[n["k_norm"]].to(torch.float32).contiguous() if self.own_keys else None
        if self.sink:
            self.sinks = tensors[n["sink"]].to(torch.float32).contiguous()
        if self.slope_exponent is not None:     # float64 powers, rounded once
            head = torch.arange(1, self.heads + 1, dtype=torch.float64)
            self.slopes = torch.pow(2.0, -self.slope_exponent * head / self.heads).to(torch.float32).to(device)
        inputs = ("q", "k", "v") if self.own_keys else ("q",)
        if self.conv:
            self.conv_weight = torch.cat([tensors[n[key + "_conv"]].to(torch.float32) for key in inputs], dim=0).contiguous()
        rows = [tensors[n[key]] for key in inputs] + ([tensors[n["g"]]] if self.gate else [])
        weight = torch.cat(rows, dim=0) if len(rows) > 1 else rows[0]
        bias = None
        if self.bias:
            bias = torch.cat([tensors["q_proj.bias"].float(), tensors["k_proj.bias"].float(), tensors["v_proj.bias"].float()])
        self.qkv = Linear(weight, bias)                # [q | k | v | gate], without k and v in a layer that reads another's cache
        self.q_only = self.qkv.rows(0, self.heads * self.head_dim) if self.own_keys and not self.gate else self.qkv
        self.out = Linear(tensors[n["o"]], tensors["o_proj.bias"] if self.bias else None)

    def projections(self) -> list:
        return [self.qkv, self.out]             # q_only is a view of qkv's first rows

    def vectors(self) -> list[torch.Tensor]:
        return [t for t in (self.q_norm, self.k_norm, self.conv_weight, self.slopes) if t is not None]

    def device_driven(self) -> bool:
        return True

    # ------------------------------------------------------------------- running
    def forward(self, ctx, x, cache, states) -> Delta:
        if cache is None or cache.k_pool is None:
            raise RuntimeError("attention needs a cache with storage")
        table = ctx.tables[cache.group]
        q_cols = self.heads * self.head_dim
        rot = self.rot
        mixed = ctx.scratch("attention.mixed", (ctx.n_tokens, self.heads * self.value_dim))
        if self.general:
            if cache.writes != self.own_keys and (self.gate or self.conv or not self.own_keys):
                raise RuntimeError("an attention layer writes the cache exactly when it projects keys and values of its own")
            projection = (self.qkv if cache.writes else self.q_only)(ctx, x, "attention.qkv")
            gate = projection[:, :, projection.shape[2] - self.gate_cols:] if self.gate else None
            source = projection[:, :, :projection.shape[2] - self.gate_cols] if self.gate else projection
            if self.conv:                          # q, k and v pass the convolution on their way from the product to the norm
                mixed_in = ctx.scratch("attention.conv", (1, ctx.n_tokens, self.conv_channels), torch.float32)
                tail = states[0] if self.conv > 1 else ctx.scratch("attention.no_tail", (1, 0, self.conv_channels), torch.float32)
                api.causal_conv(projection, 0, self.conv_channels, self.conv_weight, None, False, tail, mixed_in[0], ctx.cu, ctx.slots,
                                ctx.sequences, ctx.n_tokens, ctx.decode)
                source = mixed_in
            q = ctx.scratch("attention.q", (ctx.n_tokens, q_cols))
            # prompts: positions, cosines and sines come from the step's table, made once for all layers and heads
            cos_sin, where = self.step_rope_table(ctx) if (rot.rotary_dim and not ctx.decode) else (None, None)
            api.qk_norm_rope_append(source, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, rot.inv_freq, rot.rotary_dim,
                                    rot.interleaved, rot.attention_scaling, q, cache.k_pool if cache.writes else None,
                                    cache.v_pool if cache.writes else None, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens,
                                    self.heads, self.kv_heads, self.head_dim, self.value_dim, ctx.status, cos_sin, where)
            self.attend(ctx, q, cache, table, mixed, gate)
            return self.out.delta(ctx, mixed, "attention.out")
        if (cache.writes and not ctx.decode and x.dtype == torch.bfloat16
                and api.gemm_tcgen05_qkv_rope_takes(x, self.qkv.weight, self.head_dim, rot.rotary_dim)):
            # long prompts: the qkv product's epilogue rotates, narrows and appends to the cache, so the float32
            # product never goes to memory and back; positions, block lookups' inputs and the cosines and sines
            # are the same for every layer and are made once per step
            cos_sin, where = self.step_rope_table(ctx)
            q = ctx.scratch("attention.q", (ctx.n_tokens, q_cols))
            api.set_label("attention.qkv")
            api.gemm_tcgen05_qkv_rope(x, self.qkv.weight, self.qkv.bias, q, cache.k_pool, cache.v_pool, cos_sin, where, table, self.heads,
                                      self.kv_heads, self.head_dim, rot.attention_scaling, ctx.status)
            self.attend(ctx, q, cache, table, mixed)
            return self.out.delta(ctx, mixed, "attention.out")
        projection = (self.qkv if cache.writes else self.q_only)(ctx, x, "attention.qkv")
        splits = self.decode_slices(ctx)
        if (ctx.decode and ctx.sequences * self.kv_heads * splits <= api.sm_count(x.device)
                and api.attention_decode_rope_supports(mixed.dtype, self.heads, self.kv_heads, self.head_dim, rot.rotary_dim)):
            # decoding: rotation, cache write and attention in one kernel.  Every CTA pays the
            # rotation's latency before it can start on its keys, which is hidden while all CTAs
            # run at once (measured on a B200: 2 % faster at 32 and at 64 CTAs, 8 % slower at 512).
            part_acc, part_ml = self.slice_scratch(ctx, splits)
            api.attention_decode_rope(projection, rot.inv_freq, rot.rotary_dim, rot.attention_scaling, cache.writes,
                                      cache.k_pool, cache.v_pool, table, ctx.len_before, ctx.sequences, self.heads, self.kv_heads,
                                      self.head_dim, self.scale, self.window or 0, splits, mixed, part_acc, part_ml, ctx.status,
                                      tickets=self.tickets(ctx, splits))
            return self.out.delta(ctx, mixed, "attention.out")
        q = ctx.scratch("attention.q", (ctx.n_tokens, q_cols))
        api.rope_append(projection, rot.inv_freq, rot.rotary_dim, rot.attention_scaling, q,
                        cache.k_pool if cache.writes else None, cache.v_pool if cache.writes else None, table, ctx.cu,
                        ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads, self.kv_heads, self.head_dim, ctx.status)
        self.attend(ctx, q, cache, table, mixed)
        return self.out.delta(ctx, mixed, "attention.out")

    def step_rope_table(self, ctx):
        """(cos_sin, where) of this step for this layer's rotary table: made by the first layer that asks and kept
        in ``ctx.memo`` for the layers that share the table."""
        rot = self.rot
        key = ("rope_table", rot.signature or rot.inv_freq.data_ptr(), rot.rotary_dim)       # the model's layers usually share one table
        made = ctx.memo.get(key)
        if made is None:
            half = rot.rotary_dim // 2
            cos_sin = ctx.scratch(f"attention.rope_table.{len(ctx.memo)}", (ctx.n_tokens, half, 2), torch.float32)
            where = ctx.scratch(f"attention.rope_where.{len(ctx.memo)}", (ctx.n_tokens, 2), torch.int32)
            api.rope_table(rot.inv_freq, rot.rotary_dim, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, cos_sin, where)
            made = ctx.memo[key] = (cos_sin, where)
        return made

    def decode_slices(self, ctx) -> int:
        """Slices of the keys for the tensor-core decode kernel, which runs one CTA per (sequence, kv
        head, slice).  Measured on a B200 from 1 to 64 sequences and 2,048 to 32,768 keys: a step is
        fastest when the slices just fill one wave of one CTA per SM and keep at least 8 blocks each; a
        second wave gains nothing."""
        splits = kv_splits(ctx, ctx.sequences * self.kv_heads, 512, api.sm_count(ctx.status.device))
        return splits if not self.window else max(1, min(splits, self.window // 512))      # a window bounds the keys there are to slice

    def slice_scratch(self, ctx, splits: int):
        """Where the slices of the keys leave their partial results (nothing for one slice)."""
        if splits <= 1:
            return None, None
        return (ctx.scratch("attention.part_acc", (ctx.n_tokens * self.heads * splits * self.value_dim,), torch.float32),
                ctx.scratch("attention.part_ml", (ctx.n_tokens * self.heads * splits * 2,), torch.float32))

    def tickets(self, ctx, splits: int):
        """With more key slices than a thread-block cluster combines (8), the decode kernel's CTAs draw tickets and
        the last one of a (sequence, kv head) combines the slices: one word each, zero between launches."""
        if splits <= 8:
            return None
        return ctx.workspace.get_zeroed("attention.tickets", (max(ctx.sequences * self.kv_heads, 64),), torch.int32)

    TENSOR_CORES_FROM = 1           # packed tokens from which prompts run the tcgen05 kernel

    @property
    def shaped_scores(self) -> bool:
        """Capped scores or a distance bias: what only the exact kernel applies."""
        return self.softcap > 0.0 or self.slopes is not None

    def attend(self, ctx, q, cache, table, mixed, gate=None) -> None:
        """Prompts in bfloat16 with head size 64 or 128: the tcgen05 kernel.  Other bfloat16
        sizes up to 128 and all decoding: the mma.sync kernels.  Everything else (float32,
        head sizes 48, 80, 144 ..., values of another size than the keys): the exact kernel.
        Sinks go with the tcgen05 prompt kernel, the mma.sync decode kernel and the exact kernel."""
        same = self.value_dim == self.head_dim
        if (same and not ctx.decode and ctx.n_tokens >= self.TENSOR_CORES_FROM
                and api.attention_tcgen05_supports(q.dtype, self.heads, self.kv_heads, self.head_dim)):
            # capped scores and the distance bias are the kernel's own (its instances that shape the scores).  So could the gate
            # be, but a softmax thread owns a row and reads its gate numbers one 32-byte sector a load (measured on a B200:
            # 2,048 tokens of 16 heads of 128 took 121 us with the gate inside against 50 + 15 us with the pass below)
            api.attention_tcgen05(q, cache.k_pool, cache.v_pool, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads,
                                  self.kv_heads, self.head_dim, self.scale, self.window or 0, mixed, ctx.status, sinks=self.sinks,
                                  softcap=self.softcap, slopes=self.slopes)
            if gate is not None:
                api.sigmoid_gate(mixed, gate, self.value_dim if self.gate == "head" else 0)
            return
        tensor_cores = (same and api.attention_mma_supports(q.dtype, self.heads, self.kv_heads, self.head_dim)
                        and ((self.sinks is None and not self.shaped_scores) or ctx.decode))
        if tensor_cores:
            splits = self.decode_slices(ctx)
        else:
            splits = kv_splits(ctx, ctx.n_tokens * self.heads, 256, 8 * api.sm_count(q.device))
        part_acc, part_ml = self.slice_scratch(ctx, splits)
        if tensor_cores:
            api.attention_mma(q, cache.k_pool, cache.v_pool, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads,
                              self.kv_heads, self.head_dim, self.scale, self.window or 0, splits, mixed, part_acc, part_ml, ctx.status,
                              one_token_each=ctx.decode, tickets=self.tickets(ctx, splits) if ctx.decode else None,
                              sinks=self.sinks if ctx.decode else None, softcap=self.softcap, slopes=self.slopes)
            if gate is not None:
                api.sigmoid_gate(mixed, gate, self.value_dim if self.gate == "head" else 0)
        else:
            if self.window:                     # a window bounds the keys a slice can hold
                splits = max(1, min(splits, self.window // 64))
                part_acc, part_ml = self.slice_scratch(ctx, splits)
            api.attention(q, cache.k_pool, cache.v_pool, table, ctx.cu, ctx.len_before, ctx.sequences, ctx.n_tokens, self.heads,
                          self.kv_heads, self.head_dim, self.scale, self.window or 0, splits, mixed, part_acc, part_ml, ctx.status,
                          value_dim=self.value_dim, sinks=self.sinks, softcap=self.softcap, slopes=self.slopes, gate=gate,
                          gate_per_head=self.gate == "head")
