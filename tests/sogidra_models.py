"""Tiny Sogidra configurations with random weights for the tests, and the plain implementation's outputs for them.
The configurations differ from one another in every size; between them they cover: one head and several, groups of one
query head per key head and of several, maps of 8 to 72 numbers with values narrower, equal and wider than a key row,
differential layers with and without the growing query gain (periods of 1, 7 and 50 positions), layers that read an
earlier layer's keys (the next layer and one further on), windows shorter than a cache block, longer than one and of a
single token, blocks of 1 token, of a few, of exactly a cache block's 64 and of more tokens than the window, scores with
and without a cap, layers without a feed-forward, a model of window layers only and one of differential layers only."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _diff(heads, kv_heads, dim, vdim, scale, diff, q_temp=None, kv_from=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if q_temp:
        out["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def _win(heads, kv_heads, dim, scale, size, pool, softcap=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "mask": {"size": size, "pool": pool}}
    if softcap:
        out["softcap"] = softcap
    return out


def _ff(n):
    return None if n is None else {"kind": "dense", "ff": n}


CONFIGS = {
    # both mixers; a window (21) and blocks (5) inside the first cache block; a reader two layers on
    "a": {
        "architecture": "Sogidra", "vocab": 211, "width": 96, "max_positions": 512, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "attention", "mixer": _diff(4, 2, 24, 40, 0.2, 0.3, (0.4, 7)), "mlp": _ff(136)},
            {"type": "attention_2", "mixer": _win(3, 1, 40, 0.16, 21, 5, 8.0), "mlp": _ff(72)},
            {"type": "attention", "mixer": _diff(2, 2, 24, 40, 0.25, 0.55, (0.2, 50), kv_from=0), "mlp": None},
        ],
    },
    # window layers only: a window of more than two cache blocks with blocks of exactly 64 tokens, a window of one token
    # with blocks of one token (every earlier token is a block of its own), blocks longer than the window; no cap
    "b": {
        "architecture": "Sogidra", "vocab": 130, "width": 64, "max_positions": 400, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "attention_2", "mixer": _win(2, 2, 16, 0.3, 150, 64), "mlp": _ff(48)},
            {"type": "attention_2", "mixer": _win(4, 1, 8, 0.5, 1, 1, 3.0), "mlp": None},
            {"type": "attention_2", "mixer": _win(1, 1, 72, 0.12, 9, 30, 30.0), "mlp": _ff(100)},
        ],
    },
    # differential layers only: one head, values wider than a key row and narrower, no query gain, a gain that grows
    # with every position, a reader right behind its source and one behind that; odd width and vocabulary
    "c": {
        "architecture": "Sogidra", "vocab": 97, "width": 72, "max_positions": 300, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "attention", "mixer": _diff(1, 1, 8, 136, 0.35, 0.2), "mlp": _ff(40)},
            {"type": "attention", "mixer": _diff(6, 3, 72, 16, 0.1, 0.8, (0.5, 1)), "mlp": None},
            {"type": "attention", "mixer": _diff(3, 3, 72, 16, 0.12, 0.4, None, kv_from=1), "mlp": _ff(24)},
            {"type": "attention", "mixer": _diff(6, 3, 72, 16, 0.08, 0.1, (0.1, 3), kv_from=1), "mlp": _ff(64)},
        ],
    },
    # sizes that the tensor cores take in bfloat16 (maps of 64, values and window heads of 128), a window that ends
    # inside the second block with blocks of 16, a differential layer after the window layer that reads the first one
    "d": {
        "architecture": "Sogidra", "vocab": 160, "width": 128, "max_positions": 640, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "attention", "mixer": _diff(4, 2, 64, 128, 0.125, 0.5, (0.3, 64)), "mlp": _ff(256)},
            {"type": "attention_2", "mixer": _win(4, 2, 128, 0.09, 100, 16, 20.0), "mlp": _ff(192)},
            {"type": "attention", "mixer": _diff(2, 2, 64, 128, 0.125, 0.7, (0.3, 64), kv_from=0), "mlp": _ff(128)},
            {"type": "attention_2", "mixer": _win(2, 1, 64, 0.125, 33, 8), "mlp": None},
        ],
    },
}
SEEDS = {"a": 3, "b": 4, "c": 6, "d": 8}
# how far the query and key projections are scaled up: enough for peaked attention, not so far that the rounding of a
# query to bfloat16 alone decides which key wins (maps of 72 numbers with a gain that grows with every position)
QK_GAIN = {"a": 25.0, "b": 25.0, "c": 10.0, "d": 25.0}


def shape_weights(tensors: dict[str, torch.Tensor], seed: int, qk_gain: float = 25.0) -> dict[str, torch.Tensor]:
    """Rescale the drawn weights so that every mechanism moves the logits: hidden states and logits of order one, peaked
    attention, a second map whose weight is far from zero, biases, position vectors and activation numbers that count."""
    g = torch.Generator().manual_seed(seed + 1000)
    out = {}
    for name, t in tensors.items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if name in ("embed", "pos"):
            t = t * 30.0
        elif leaf in ("mix.q", "mix.k"):
            t = t * qk_gain
        elif leaf.endswith(".b"):
            t = torch.randn(t.shape, generator=g) * 0.5
        elif leaf in ("mix.lq1", "mix.lk1", "mix.lq2", "mix.lk2"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif leaf == "mlp.act":
            t = torch.randn(t.shape, generator=g)
        elif leaf == "dwa" or "norm" in leaf:
            pass
        elif leaf.startswith("mix.") or leaf.startswith("mlp."):
            t = t * 10.0
        out[name] = t
    return out


def write_model(folder: Path, name: str, stored: str = "float32") -> Path:
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel
    from thintensor_b200.weights.random_init import STORED_DTYPES, random_tensors
    from thintensor_b200.weights.safetensors_io import write_safetensors

    arch, config = load_config(CONFIGS[name])
    declared = DecoderModel(arch.describe(config), torch.float32, None).weight_declarations()
    tensors = shape_weights(random_tensors(declared, SEEDS[name], torch.float32), SEEDS[name], QK_GAIN[name])
    tensors = {k: v.to(STORED_DTYPES[stored]) for k, v in tensors.items()}
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(CONFIGS[name], indent=1))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


_oracle: dict = {}


def oracle_logits(folder: Path, tokens: list[int]) -> torch.Tensor:
    """float64 logits [T, vocab] of the plain implementation for one whole sequence."""
    import plain_sogidra

    model_key = ("model", str(folder))
    if model_key not in _oracle:
        _oracle[model_key] = plain_sogidra.read_model(folder)
    key = (str(folder), tuple(tokens))
    if key not in _oracle:
        cfg, weights = _oracle[model_key]
        with torch.no_grad():
            _oracle[key] = plain_sogidra.forward(cfg, weights, tokens)
    return _oracle[key]


def oracle_sensitivity(folder: Path, tokens: list[int]) -> torch.Tensor:
    """Per position, one minus the cosine between the plain implementation's logits and its logits with every operand of
    a matrix product and every cached number narrowed to bfloat16 on the way, everything else as exact as before: how far
    rounding alone carries that position."""
    import plain_sogidra

    key = ("sensitivity", str(folder), tuple(tokens))
    if key not in _oracle:
        want = oracle_logits(folder, tokens)
        cfg, weights = _oracle[("model", str(folder))]
        with torch.no_grad():
            other = plain_sogidra.forward(cfg, weights, tokens, narrow=lambda x: x.to(torch.bfloat16).to(x.dtype))
        _oracle[key] = 1.0 - torch.nn.functional.cosine_similarity(want, other, dim=-1)
    return _oracle[key]


def oracle_float32_drift(folder: Path, tokens: list[int]) -> torch.Tensor:
    """Per position, the largest difference between the plain implementation's logits and its logits with every operand of
    a matrix product and every cached number rounded to float32 on the way: where a differential layer subtracts two
    nearly equal maps before its norm, float32 rounding alone is carried this far."""
    import plain_sogidra

    key = ("drift", str(folder), tuple(tokens))
    if key not in _oracle:
        want = oracle_logits(folder, tokens)
        cfg, weights = _oracle[("model", str(folder))]
        with torch.no_grad():
            other = plain_sogidra.forward(cfg, weights, tokens, narrow=lambda x: x.to(torch.float32).to(x.dtype))
        _oracle[key] = (want - other).abs().max(dim=-1).values
    return _oracle[key]
