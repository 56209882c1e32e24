"""The Kerepel decoder as a description: which parts each layer has, with what numbers, and what the
checkpoint calls their tensors.

Layers are pre-norm with RMS norms (``l<i>.norm1``, ``l<i>.norm2``); the mixer's tensors lie under ``l<i>.mix.`` (``q``, ``k``,
``v``, ``g``, ``o``, the convolutions ``q.conv`` / ..., the per-head norms ``q.norm`` / ``k.norm``; for latent attention ``q``,
``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``g``, ``o``), the feed-forward's under ``l<i>.mlp.`` (``up`` / ``down``, or ``e<k>.gate`` /
``up`` / ``down``, ``router``, ``correction``, ``shared.gate`` / ... / ``shared.sg``), the layer's token side input under
``l<i>.side.`` with the table ``side.embed`` shared by all layers.  The token table is ``embed`` (also the output matrix),
the hashed pair table ``bigram``, the last norm ``final.norm``.

What the design fixes lives here: the slopes of the distance bias are ``2 ** (-8 (h + 1) / heads)``, the experts' unit uses
``sigmoid(1.702 g)``, routing scores are sigmoids with a correction for the choice, groups are scored by their two best and
the weights are not renormalised, the rotation pairs neighbours with YaRN frequencies.
"""
from __future__ import annotations

from ..config.kerepel import ARCHITECTURE, AttentionSizes, DenseSizes, KerepelConfig, LatentAttentionSizes, MoeSizes
from ..config.registry import Architecture, register_architecture
from ..parts.rope import yarn_attention_scaling
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_norm": "q.norm", "k_norm": "k.norm", "q_conv": "q.conv",
                   "k_conv": "k.conv", "v_conv": "v.conv"}
LATENT_NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "g": "g", "o": "o"}
MLP_NAMES = {"up": "up", "down": "down"}
MOE_NAMES = {"router": "router", "expert": "e{}.", "shared": "shared.", "gate": "gate", "up": "up", "down": "down",
             "correction": "correction", "shared_gate": "shared.sg"}
SLOPE_EXPONENT = 8.0
EXPERT_ALPHA = 1.702


def attention_part(config: KerepelConfig, sizes: AttentionSizes, prefix: str, cache_window: int | None) -> PartSpec:
    return PartSpec("attention", {
        "hidden": config.width, "heads": sizes.heads, "kv_heads": sizes.kv_heads, "head_dim": sizes.dim, "value_dim": sizes.vdim,
        "scale": sizes.scale, "window": sizes.window, "qk_norm_eps": config.eps, "conv": sizes.conv, "softcap": sizes.softcap,
        "slope_exponent": SLOPE_EXPONENT, "gate": "elementwise", "own_keys": sizes.kv_from is None, "cache_window": cache_window,
        "names": ATTENTION_NAMES}, prefix)


def latent_attention_part(config: KerepelConfig, sizes: LatentAttentionSizes, prefix: str) -> PartSpec:
    position = None
    if sizes.rot is not None:
        scaling, factor = None, 1.0
        if sizes.rot.scaling is not None:
            s = sizes.rot.scaling
            scaling = {"rope_type": "yarn", "factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            factor = yarn_attention_scaling(s.factor)
        position = PartSpec("rope", {"head_dim": sizes.rot_dim, "theta": sizes.rot.base, "rotary_dim": sizes.rot.dims, "scaling": scaling,
                                     "attention_scaling": factor, "interleaved": True, "table_precision": "float64"})
    return PartSpec("latent_attention", {
        "hidden": config.width, "heads": sizes.heads, "dim": sizes.dim, "rot_dim": sizes.rot_dim, "value_dim": sizes.vdim, "q_rank": None,
        "kv_rank": sizes.kv_rank, "scale": sizes.scale, "eps": config.eps, "position": position, "gate": "head", "names": LATENT_NAMES},
        prefix)


def feed_forward_part(config: KerepelConfig, sizes, prefix: str) -> PartSpec:
    if isinstance(sizes, DenseSizes):
        return PartSpec("mlp", {"hidden": config.width, "inter": sizes.ff, "activation": "gelu", "names": MLP_NAMES}, prefix)
    assert isinstance(sizes, MoeSizes)
    return PartSpec("moe", {
        "hidden": config.width, "experts": sizes.experts, "top": sizes.top, "inter": sizes.ff, "groups": sizes.groups, "keep": sizes.keep,
        "shared_inter": sizes.shared_ff, "activation": "clamped", "limit": sizes.limit, "shared_limit": sizes.shared_limit,
        "alpha": EXPERT_ALPHA, "score": "sigmoid", "correction": True, "group_score": "top2", "renormalize": False,
        "shared_gate": bool(sizes.shared_ff), "names": MOE_NAMES}, prefix)


def describe_kerepel(config: KerepelConfig) -> ModelSpec:
    def norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": config.width, "eps": config.eps, "name": name}, prefix)

    # a layer whose cache others read keeps what the widest of their windows sees
    reach: dict[int, int | None] = {}
    for layer in config.layers:
        if layer.type == "attention" and layer.mixer.kv_from is not None:
            source, mine = layer.mixer.kv_from, layer.mixer.window
            known = reach.get(source, config.layers[source].mixer.window)
            reach[source] = None if known is None or mine is None else max(known, mine)

    count = len(config.layers)
    layers, schedule = [], []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        parts = {"mixer_norm": norm(prefix, "norm1")}
        source = None
        if layer.type == "attention":
            sizes = layer.mixer
            cache_window = None                 # the layer's own window
            if index in reach:
                cache_window = -1 if reach[index] is None else reach[index]
            parts["mixer"] = attention_part(config, sizes, prefix + "mix.", cache_window)
            source = sizes.kv_from
        else:
            parts["mixer"] = latent_attention_part(config, layer.mixer, prefix + "mix.")
        if layer.mlp is not None:
            parts["ffn_norm"] = norm(prefix, "norm2")
            parts["ffn"] = feed_forward_part(config, layer.mlp, prefix + "mlp.")
        if config.side_dim:
            parts["side"] = PartSpec("token_side", {
                "hidden": config.width, "vocab": config.vocab, "dim": config.side_dim, "table_cols": count * config.side_dim,
                "offset": index * config.side_dim, "eps": config.eps,
                "names": {"table": "side.embed", "gate": prefix + "side.gate", "proj": prefix + "side.proj", "norm": prefix + "side.norm"}}, "")
        layers.append(LayerSpec("pre_norm", parts))
        schedule.append(Run(index, source))
    if config.bigram is not None:
        embedding = PartSpec("table_pair_hash", {"vocab": config.vocab, "hidden": config.width, "buckets": config.bigram.buckets,
                                                 "mul_prev": config.bigram.mul_prev, "mul_cur": config.bigram.mul_cur, "name": "embed",
                                                 "pair_name": "bigram"}, "")
    else:
        embedding = PartSpec("table", {"vocab": config.vocab, "hidden": config.width, "name": "embed"}, "")
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        embedding=embedding,
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.", "norm"),
        head=PartSpec("linear", {"hidden": config.width, "vocab": config.vocab, "name": "head", "fallback": "embed", "tied": True,
                                 "scale": 1.0 if config.logit_scale is None else config.logit_scale}, ""),
    )


register_architecture(Architecture(
    name=ARCHITECTURE,
    model_types=("kerepel",),
    config_class=KerepelConfig,
    describe=describe_kerepel,
))
