"""The Sogidra decoder as a description: which parts each layer has, with what numbers, and what the
checkpoint calls their tensors.

The token table is ``embed`` (also the output matrix), the learned position table ``pos``, the last norm
``final.norm``.  Layer ``i``'s tensors start with ``l<i>.``: the norms before and after the mixer (``norm1``,
``norm1b``) and before and after the feed-forward (``norm2``, ``norm2b``), all RMS norms whose stored weight is the
distance from one; the mixer's tensors under ``mix.``, the feed-forward's under ``mlp.`` (``up``, ``down`` and the two
numbers ``act`` of its activation); and ``dwa``, the weights with which the layer's end mixes the embedding's output
and every layer's result so far.  A differential layer that reads another layer's keys and values stores no ``k`` and
``v`` tensors and its run of the schedule reads that layer's cache.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.sogidra import ARCHITECTURE, DifferentialSizes, PooledWindowSizes, SogidraConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

DIFFERENTIAL_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                      "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}
WINDOW_NAMES = {"q": "q", "k": "k", "o": "o"}
FFN_NAMES = {"up": "up", "down": "down", "act": "act"}


def differential_part(config: SogidraConfig, sizes: DifferentialSizes, prefix: str) -> PartSpec:
    return PartSpec("differential_attention", {
        "hidden": config.width, "heads": sizes.heads, "kv_heads": sizes.kv_heads, "dim": sizes.dim, "value_dim": sizes.vdim,
        "scale": sizes.scale, "diff": sizes.diff, "eps": config.eps, "bias": True,
        "q_gain": None if sizes.q_temp is None else (sizes.q_temp.coef, sizes.q_temp.every),
        "own_keys": sizes.kv_from is None, "names": DIFFERENTIAL_NAMES}, prefix)


def window_part(config: SogidraConfig, sizes: PooledWindowSizes, prefix: str) -> PartSpec:
    return PartSpec("pooled_window_attention", {
        "hidden": config.width, "heads": sizes.heads, "kv_heads": sizes.kv_heads, "dim": sizes.dim, "scale": sizes.scale,
        "softcap": sizes.softcap, "eps": config.eps, "window": sizes.window, "pool": sizes.pool, "names": WINDOW_NAMES}, prefix)


def describe_sogidra(config: SogidraConfig) -> ModelSpec:
    def norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": config.width, "eps": config.eps, "weight_offset": 1.0, "name": name, "init": "zeros"}, prefix)

    layers, schedule = [], []
    count = len(config.layers) + 1              # results that the layers' ends mix: the embedding's output and one per layer
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        parts = {"mixer_norm": norm(prefix, "norm1"), "mixer_post_norm": norm(prefix, "norm1b")}
        if layer.type == "attention":
            parts["mixer"] = differential_part(config, layer.mixer, prefix + "mix.")
        else:
            parts["mixer"] = window_part(config, layer.mixer, prefix + "mix.")
        if layer.ff is not None:
            parts["ffn_norm"] = norm(prefix, "norm2")
            parts["ffn"] = PartSpec("mlp", {"hidden": config.width, "inter": layer.ff, "activation": "xielu", "names": FFN_NAMES}, prefix + "mlp.")
            parts["ffn_post_norm"] = norm(prefix, "norm2b")
        parts["depth"] = PartSpec("weighted_results", {"count": index + 2, "name": "dwa"}, prefix)
        layers.append(LayerSpec("sandwich", parts, {"result_index": index + 1, "results": count}))
        schedule.append(Run(index, cache_from=layer.mixer.kv_from if layer.type == "attention" else None))
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        embedding=PartSpec("table_positions", {"vocab": config.vocab, "hidden": config.width, "positions": config.max_positions,
                                               "name": "embed", "position_name": "pos"}, ""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.", "norm"),
        head=PartSpec("linear", {"hidden": config.width, "vocab": config.vocab, "fallback": "embed", "tied": True, "name": "head"}, ""),
    )


register_architecture(Architecture(
    name=ARCHITECTURE,
    model_types=("sogidra",),
    config_class=SogidraConfig,
    describe=describe_sogidra,
))
