"""Tiny Kerepel configurations with random weights for the tests, the plain implementation's outputs for them, and the
judge that compares an engine's logits with those.  The configurations differ from one another in every size; between
them they cover: one key/value head for all query heads and one for each, key and value sizes that differ, windows that
end inside the first cache block, span more than two blocks and are absent, readers of another layer's keys with a wider
and with a narrower window than their source and with other convolution taps, convolutions of 2, 3 and 4 taps and none,
capped and uncapped scores, latents smaller and larger than the heads they expand into, a rotation with and without YaRN
scaling and none, dense feed-forwards whose width is no multiple of four, experts in groups of two and three and
ungrouped, one choice and several, limits below and above one, layers with and without a shared expert and without any
feed-forward, a model without pair table, side input and logit scale, and one whose heads have tensor-core sizes."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _moe(experts, top, ff, limit, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def _yarn(dims, base, factor=None, original=None, fast=None, slow=None):
    rot = {"dims": dims, "base": base}
    if factor:
        rot["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return rot


CONFIGS = {
    # the source's window (21) ends inside the first block; its reader looks further back (40) with other taps
    "a": {
        "architecture": "Kerepel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.75,
        "embedding": {"bigram": {"buckets": 97, "mul_prev": 5, "mul_cur": 11}}, "token_side": {"dim": 8},
        "layers": [
            {"type": "attention", "mlp": {"kind": "dense", "ff": 136}, "mixer": {
                "heads": 3, "kv_heads": 3, "dim": 16, "vdim": 24, "conv": 4, "mask": {"size": 21}, "scale": 0.3, "softcap": 30.0}},
            {"type": "latent_attention", "mlp": _moe(6, 2, 40, 1.5, (3, 2), (24, 0.75)), "mixer": {
                "heads": 2, "dim": 24, "rot_dim": 8, "vdim": 16, "kv_rank": 40, "scale": 0.2, "rot": _yarn(8, 1000.0, 4.0, 32, 8.0, 1.0)}},
            {"type": "attention", "mlp": None, "mixer": {
                "heads": 3, "kv_heads": 3, "dim": 16, "vdim": 24, "conv": 2, "kv_from": 0, "mask": {"size": 40}, "scale": 0.25, "softcap": 20.0}},
        ],
    },
    # nothing optional: no pair table, no side input, no logit scale; a window over more than two blocks; a reader with
    # a narrower window and no cap; a dense width that is no multiple of four; one latent head; groups of two
    "b": {
        "architecture": "Kerepel", "vocab": 130, "width": 64, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "latent_attention", "mlp": _moe(8, 3, 16, 1.0, (4, 2)), "mixer": {
                "heads": 1, "dim": 48, "rot_dim": 16, "vdim": 8, "kv_rank": 24, "scale": 0.15, "rot": _yarn(16, 500.0)}},
            {"type": "attention", "mlp": {"kind": "dense", "ff": 102}, "mixer": {
                "heads": 4, "kv_heads": 1, "dim": 32, "vdim": 32, "conv": 2, "mask": {"size": 150}, "scale": 0.2, "softcap": 50.0}},
            {"type": "attention", "mlp": _moe(5, 5, 24, 2.0, None, (12, 2.5)), "mixer": {
                "heads": 4, "kv_heads": 1, "dim": 32, "vdim": 32, "conv": 3, "kv_from": 1, "mask": {"size": 70}, "scale": 0.17}},
        ],
    },
    # heads of tensor-core sizes; attention without a window and without a convolution; a latent layer without rotation;
    # experts of which one is chosen; groups the size of one expert
    "c": {
        "architecture": "Kerepel", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 2.0,
        "embedding": {"bigram": {"buckets": 61, "mul_prev": 3, "mul_cur": 1}}, "token_side": {"dim": 16},
        "layers": [
            {"type": "attention", "mlp": {"kind": "dense", "ff": 96}, "mixer": {
                "heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "conv": 3, "mask": {"size": 100}, "scale": 0.125, "softcap": 40.0}},
            {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 192}, "mixer": {
                "heads": 2, "dim": 32, "rot_dim": 32, "vdim": 64, "kv_rank": 48, "scale": 0.13, "rot": _yarn(32, 10000.0, 2.0, 64, 16.0, 2.0)}},
            {"type": "attention", "mlp": {"kind": "dense", "ff": 64}, "mixer": {
                "heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09, "softcap": 25.0}},
            # the one-choice routing stands last: a close call that rounding decides the other way moves its own position only
            {"type": "latent_attention", "mlp": _moe(4, 1, 48, 0.5, (4, 2), (64, 1.0)), "mixer": {
                "heads": 3, "dim": 96, "rot_dim": 32, "vdim": 128, "kv_rank": 72, "scale": 0.1}},
        ],
    },
}
SEEDS = {"a": 3, "b": 4, "c": 6}


def shape_weights(tensors: dict[str, torch.Tensor], seed: int) -> dict[str, torch.Tensor]:
    """Rescale the drawn weights so that every mechanism moves the logits: hidden states and logits of order one, peaked
    attention, gates and routers away from their middle, clamps that bite, corrections that change the choice."""
    out = {}
    for name, t in tensors.items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if name in ("embed", "bigram"):
            t = t * 30.0
        elif name == "side.embed":
            t = t * 50.0
        elif leaf.endswith(".conv"):
            t = t * 5.0
        elif leaf in ("mix.q", "mix.k", "mix.dkv"):
            t = t * 25.0
        elif leaf.endswith("router") or leaf.endswith("shared.sg"):
            t = t * 8.0             # sigmoid scores spread over (0, 1): saturated ones would leave the choice to their last bits
        elif leaf.endswith("correction"):
            t = t * 3.0
        elif "norm" in leaf:
            pass
        elif leaf.startswith("mix.") or leaf.startswith("mlp.") or leaf.startswith("side."):
            t = t * 10.0
        out[name] = t
    return out


def write_model(folder: Path, name: str, stored: str = "float32", config: dict | None = None, seed: int | None = None) -> Path:
    from thintensor_b200.config.registry import load_config
    from thintensor_b200.engine.model import DecoderModel
    from thintensor_b200.weights.random_init import STORED_DTYPES, random_tensors
    from thintensor_b200.weights.safetensors_io import write_safetensors

    config = CONFIGS[name] if config is None else config
    seed = SEEDS[name] if seed is None else seed
    arch, typed = load_config(config)
    declared = DecoderModel(arch.describe(typed), torch.float32, None).weight_declarations()
    tensors = shape_weights(random_tensors(declared, seed, torch.float32), seed)
    tensors = {k: v.to(STORED_DTYPES[stored]) for k, v in tensors.items()}
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


_oracle: dict = {}


def oracle_logits(folder: Path, tokens: list[int]) -> torch.Tensor:
    """float64 logits [T, vocab] of the plain implementation for one whole sequence."""
    import plain_kerepel

    model_key = ("model", str(folder))
    if model_key not in _oracle:
        _oracle[model_key] = plain_kerepel.read_model(folder)
    key = (str(folder), tuple(tokens))
    if key not in _oracle:
        cfg, weights = _oracle[model_key]
        with torch.no_grad():
            _oracle[key] = plain_kerepel.forward(cfg, weights, tokens)
    return _oracle[key]


def oracle_sensitivity(folder: Path, tokens: list[int]) -> torch.Tensor:
    """Per position, one minus the cosine between the plain implementation's logits and its logits with every operand of
    a matrix product narrowed to bfloat16 on the way: how far the rounding of activations alone carries that position."""
    import plain_kerepel

    key = ("sensitivity", str(folder), tuple(tokens))
    if key not in _oracle:
        want = oracle_logits(folder, tokens)
        cfg, weights = _oracle[("model", str(folder))]
        with torch.no_grad():
            other = plain_kerepel.forward(cfg, weights, tokens, narrow=lambda x: x.to(torch.bfloat16).to(x.dtype))
        _oracle[key] = 1.0 - torch.nn.functional.cosine_similarity(want, other, dim=-1)
    return _oracle[key]


class Judge:
    """Compares rows of logits with the plain implementation's.  float32: every logit within 5e-5 of the request's largest
    one.  bfloat16: the cosine with the plain logits, position by position, against ``1 - cos <= 1e-3 + 4 s``, s being how
    far the plain implementation itself moves at that position when it narrows its activations to bfloat16.  A router's
    close call can fall the other way under the engine's rounding, which moves that position without any fault; so over a
    test up to one position in twenty-five (and one) may exceed its bound, while the mean of ``1 - cos`` stays within 0.01
    of the mean bound."""

    def __init__(self, dtype, folder):
        self.dtype, self.folder, self.away, self.over, self.notes, self.bounds = dtype, folder, [], 0, [], []

    def add(self, got, tokens, rows, what):
        rows = list(rows)
        want = oracle_logits(self.folder, tokens)[rows]
        got = got.double().cpu().reshape(-1, got.shape[-1])
        assert got.shape == want.shape and torch.isfinite(got).all(), what
        if self.dtype == "float32":
            scale = max(1.0, float(want.abs().max()))
            err = (got - want).abs().max(dim=-1).values
            worst = int(err.argmax())
            assert float(err[worst]) <= 5e-5 * scale, f"{what}: position {rows[worst]}: max |diff| {float(err[worst]):.3e} with logits up to {scale:.3f}"
            return
        away = 1.0 - torch.nn.functional.cosine_similarity(got, want, dim=-1)
        bound = 1e-3 + 4.0 * oracle_sensitivity(self.folder, tokens)[rows]
        bad = away > bound
        if bool(bad.any()):
            worst = int((away / bound).argmax())
            self.notes.append(f"{what}: position {rows[worst]} has cosine {1 - float(away[worst]):.5f}, rounding alone allows {1 - float(bound[worst]):.5f}")
        self.over += int(bad.sum())
        self.away.append(away)
        self.bounds.append(bound)

    def done(self):
        if self.dtype == "bfloat16":
            away = torch.cat(self.away)
            assert self.over <= 1 + away.numel() // 25, f"{self.over} of {away.numel()} positions beyond their bound; " + "; ".join(self.notes[:4])
            allowed = 0.01 + float(torch.cat(self.bounds).mean())
            assert float(away.mean()) <= allowed, f"mean cosine {float(1.0 - away.mean()):.5f}, rounding alone allows {1.0 - allowed:.5f}"
