"""Typed configuration of the Sogidra decoder, read from its config.json.

config.json gives ``vocab``, ``width``, ``max_positions`` (rows of the learned position table), ``norm.eps`` and
``layers``: a list whose entries name the layer's mixer (``type``: ``attention``, the differential attention, or
``attention_2``, the window attention with pooled blocks), the mixer's sizes (``mixer``) and the feed-forward
(``mlp``: ``{"kind": "dense", "ff": n}``, or null for a layer without one).  A differential mixer may name an earlier
layer whose keys and values it reads (``kv_from``) and may scale its queries with the position (``q_temp``: ``coef``,
``every``); a window mixer gives its window and block size (``mask``: ``size``, ``pool``) and may cap its scores
(``softcap``).  Every size and constant of a model is one of these numbers; the code holds only what the design fixes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError
from .famalorn import _float, _int

ARCHITECTURE = "Sogidra"
MIXER_TYPES = ("attention", "attention_2")


def _heads(raw: dict, where: str) -> tuple[int, int]:
    heads, kv_heads = _int(raw, "heads", where), _int(raw, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: {heads} query heads are not a multiple of {kv_heads} key/value heads")
    return heads, kv_heads


@dataclass(frozen=True)
class QueryTemperature:
    """Queries at position p are multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``."""

    coef: float
    every: int

    def to_dict(self) -> dict:
        return {"coef": self.coef, "every": self.every}


@dataclass(frozen=True)
class DifferentialSizes:
    heads: int
    kv_heads: int
    dim: int                # query/key numbers per head and map (a head's row holds two maps)
    vdim: int
    scale: float
    diff: float             # the constant of the second map's weight, and one minus the output's gain
    q_temp: QueryTemperature | None = None
    kv_from: int | None = None      # the layer whose keys and values this one reads

    @staticmethod
    def from_dict(raw: dict, where: str) -> "DifferentialSizes":
        heads, kv_heads = _heads(raw, where)
        temp = raw.get("q_temp")
        source = raw.get("kv_from")
        return DifferentialSizes(
            heads, kv_heads, _int(raw, "dim", where), _int(raw, "vdim", where), _float(raw, "scale", where), _float(raw, "diff", where),
            QueryTemperature(_float(temp, "coef", where + ".q_temp"), _int(temp, "every", where + ".q_temp")) if temp else None,
            None if source is None else _int(raw, "kv_from", where, 0))

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"diff": self.diff, "dim": self.dim, "heads": self.heads}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        out["kv_heads"] = self.kv_heads
        if self.q_temp is not None:
            out["q_temp"] = self.q_temp.to_dict()
        out.update({"scale": self.scale, "vdim": self.vdim})
        return out


@dataclass(frozen=True)
class PooledWindowSizes:
    heads: int
    kv_heads: int
    dim: int                # query/key numbers per head; the values are the keys before their norm, so as many
    scale: float
    window: int             # mask.size: a position sees itself and the window - 1 before it
    pool: int               # mask.pool: tokens of a block; whole blocks before the window are seen as their means
    softcap: float | None = None

    @staticmethod
    def from_dict(raw: dict, where: str) -> "PooledWindowSizes":
        heads, kv_heads = _heads(raw, where)
        mask = raw.get("mask")
        if not isinstance(mask, dict):
            raise ConfigError(f"config.json: {where} needs 'mask' with its window 'size' and block size 'pool'")
        dim = _int(raw, "dim", where)
        if raw.get("vdim") is not None and int(raw["vdim"]) != dim:
            raise ConfigError(f"config.json: {where}: the values are the keys, so 'vdim' must equal 'dim' ({dim}), got {raw['vdim']}")
        cap = raw.get("softcap")
        sizes = PooledWindowSizes(heads, kv_heads, dim, _float(raw, "scale", where), _int(mask, "size", where + ".mask"),
                                  _int(mask, "pool", where + ".mask"), None if not cap else float(cap))
        if sizes.softcap is not None and sizes.softcap <= 0:
            raise ConfigError(f"config.json: {where}: 'softcap' must be positive, got {sizes.softcap}")
        return sizes

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                               "mask": {"pool": self.pool, "size": self.window}, "scale": self.scale}
        if self.softcap is not None:
            out["softcap"] = self.softcap
        out["vdim"] = self.dim
        return out


@dataclass(frozen=True)
class SogidraLayer:
    type: str
    mixer: Any              # DifferentialSizes or PooledWindowSizes
    ff: int | None          # None: the layer has no feed-forward

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.ff is None else {"ff": self.ff, "kind": "dense"}, "type": self.type}


@dataclass(frozen=True)
class SogidraConfig:
    vocab: int
    width: int
    eps: float
    max_positions: int
    layers: tuple[SogidraLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(raw: dict[str, Any]) -> "SogidraConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json is missing the 'norm' entry with its eps")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        layers: list[SogidraLayer] = []
        for index, entry in enumerate(entries):
            where = f"layers[{index}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where} has type {kind!r}; known: {', '.join(MIXER_TYPES)}")
            if not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs the sizes of its mixer")
            if kind == "attention":
                mixer = DifferentialSizes.from_dict(entry["mixer"], where + ".mixer")
                if mixer.kv_from is not None:
                    source = layers[mixer.kv_from] if mixer.kv_from < index else None
                    if source is None or source.type != "attention" or source.mixer.kv_from is not None:
                        raise ConfigError(f"config.json: {where}.mixer: 'kv_from' must name an earlier differential layer that projects "
                                          f"its own keys and values, got {mixer.kv_from}")
                    theirs = source.mixer
                    if (theirs.kv_heads, theirs.dim, theirs.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                        raise ConfigError(f"config.json: {where}.mixer reads the keys and values of layer {mixer.kv_from}, whose "
                                          f"key/value heads or sizes differ")
            else:
                mixer = PooledWindowSizes.from_dict(entry["mixer"], where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None and (not isinstance(mlp, dict) or mlp.get("kind") != "dense"):
                raise ConfigError(f"config.json: {where}.mlp must be null or of kind 'dense'")
            layers.append(SogidraLayer(kind, mixer, None if mlp is None else _int(mlp, "ff", where + ".mlp")))
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return SogidraConfig(_int(raw, "vocab", "the model"), _int(raw, "width", "the model"), _float(norm, "eps", "norm"),
                             _int(raw, "max_positions", "the model"), tuple(layers), eos_ids)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "layers": [layer.to_dict() for layer in self.layers],
                               "max_positions": self.max_positions, "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
