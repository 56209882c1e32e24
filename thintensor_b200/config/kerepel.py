"""Typed configuration of the Kerepel decoder, read from its config.json.

config.json gives ``vocab``, ``width``, ``norm.eps``, ``logit_scale`` (the logits' factor; absent: 1), ``embedding.bigram``
(``buckets``, ``mul_prev``, ``mul_cur``: the hashed pair table that is added to the token embedding; absent: none),
``token_side.dim`` (numbers per layer of the second token embedding that every layer's end reads; absent: none) and
``layers``: a list whose entries name the layer's mixer (``type``: ``attention`` or ``latent_attention``), the mixer's sizes
(``mixer``) and the feed-forward (``mlp``: ``{"kind": "dense", "ff": n}``, ``{"kind": "moe", "expert": {"ff": n, "limit": c},
"router": {"experts": E, "top": k, "groups": {"count": g, "keep": m}}, "shared": {"ff": n, "limit": c}}``, or null for a
layer without one).  An attention mixer may name an earlier layer whose keys and values it reads (``kv_from``).  Every size
and constant of a model is one of these numbers; the code holds only what the design fixes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError
from .famalorn import _float, _int
from .neruzen import PairTable

ARCHITECTURE = "Kerepel"


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self) -> dict:
        original = int(self.original) if float(self.original).is_integer() else self.original
        return {"factor": self.factor, "fast": self.fast, "original": original, "slow": self.slow}


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: YarnScaling | None = None

    @staticmethod
    def from_dict(raw, where: str, most: int) -> "Rotation | None":
        if not raw:
            return None
        scaling = None
        if raw.get("scaling"):
            s, at = raw["scaling"], where + ".scaling"
            scaling = YarnScaling(_float(s, "factor", at), _float(s, "original", at), _float(s, "fast", at), _float(s, "slow", at))
            if scaling.factor <= 0 or scaling.original <= 0 or scaling.fast <= 0 or scaling.slow <= 0:
                raise ConfigError(f"config.json: {at}: factor, original, fast and slow are positive")
        rot = Rotation(_int(raw, "dims", where), _float(raw, "base", where), scaling)
        if rot.dims % 2 or rot.dims > most:
            raise ConfigError(f"config.json: {where}: the rotated part must be even and at most {most}, got {rot.dims}")
        return rot

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = self.scaling.to_dict()
        return out


@dataclass(frozen=True)
class AttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int | None            # taps of the short convolution on q, k and v; None: none
    window: int | None          # mask.size: a position sees itself and the window - 1 before it; None: all
    softcap: float | None
    kv_from: int | None = None  # the layer whose keys and values this one reads

    @staticmethod
    def from_dict(raw: dict, where: str) -> "AttentionSizes":
        mask = raw.get("mask")
        heads = _int(raw, "heads", where)
        sizes = AttentionSizes(
            heads, _int(raw, "kv_heads", where) if raw.get("kv_heads") is not None else heads, _int(raw, "dim", where),
            _int(raw, "vdim", where), _float(raw, "scale", where), _int(raw, "conv", where) if raw.get("conv") else None,
            _int(mask, "size", where + ".mask") if mask else None, _float(raw, "softcap", where) if raw.get("softcap") else None,
            _int(raw, "kv_from", where, 0) if raw.get("kv_from") is not None else None)
        if sizes.heads % sizes.kv_heads:
            raise ConfigError(f"config.json: {where}: {sizes.heads} query heads are not a multiple of {sizes.kv_heads} key/value heads")
        return sizes

    def to_dict(self) -> dict:
        out: dict[str, Any] = {}
        if self.conv is not None:
            out["conv"] = self.conv
        out.update({"dim": self.dim, "heads": self.heads})
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        out["kv_heads"] = self.kv_heads
        if self.window is not None:
            out["mask"] = {"size": self.window}
        out["scale"] = self.scale
        if self.softcap is not None:
            out["softcap"] = self.softcap
        out["vdim"] = self.vdim
        return out


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int                # unrotated query/key numbers per head
    rot_dim: int            # rotated query/key numbers per head; the key's are shared by all heads
    vdim: int
    kv_rank: int
    scale: float
    rot: Rotation | None

    @staticmethod
    def from_dict(raw: dict, where: str) -> "LatentAttentionSizes":
        rot_dim = _int(raw, "rot_dim", where)
        return LatentAttentionSizes(_int(raw, "heads", where), _int(raw, "dim", where), rot_dim, _int(raw, "vdim", where),
                                    _int(raw, "kv_rank", where), _float(raw, "scale", where),
                                    Rotation.from_dict(raw.get("rot"), where + ".rot", rot_dim))

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        out.update({"rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim})
        return out


@dataclass(frozen=True)
class DenseSizes:
    ff: int

    def to_dict(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class MoeSizes:
    experts: int
    top: int
    ff: int
    limit: float            # the experts' clamp; 0: none
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0      # 0: no shared expert
    shared_limit: float = 0.0
    grouped: bool = True    # whether config.json spells the groups out

    @staticmethod
    def from_dict(raw: dict, where: str) -> "MoeSizes":
        router, expert = raw.get("router"), raw.get("expert")
        if not isinstance(router, dict) or not isinstance(expert, dict):
            raise ConfigError(f"config.json: {where} needs 'router' and 'expert'")
        groups = router.get("groups") or {}
        shared = raw.get("shared") or {}
        sizes = MoeSizes(_int(router, "experts", where + ".router"), _int(router, "top", where + ".router"), _int(expert, "ff", where + ".expert"),
                         _float(expert, "limit", where + ".expert") if expert.get("limit") is not None else 0.0,
                         _int(groups, "count", where + ".router.groups") if groups else 1,
                         _int(groups, "keep", where + ".router.groups") if groups else 1,
                         _int(shared, "ff", where + ".shared") if shared else 0,
                         _float(shared, "limit", where + ".shared") if shared and shared.get("limit") is not None else 0.0, bool(groups))
        if sizes.experts % sizes.groups or sizes.keep > sizes.groups:
            raise ConfigError(f"config.json: {where}: {sizes.experts} experts do not form {sizes.groups} equal groups of which {sizes.keep} stay")
        if sizes.top > sizes.keep * (sizes.experts // sizes.groups):
            raise ConfigError(f"config.json: {where}: top {sizes.top} is more than the experts of {sizes.keep} groups")
        return sizes

    def to_dict(self) -> dict:
        router: dict[str, Any] = {"experts": self.experts}
        if self.grouped:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        router["top"] = self.top
        expert: dict[str, Any] = {"ff": self.ff}
        if self.limit:
            expert["limit"] = self.limit
        out: dict[str, Any] = {"expert": expert, "kind": "moe", "router": router}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff, **({"limit": self.shared_limit} if self.shared_limit else {})}
        return out


MIXER_TYPES = ("attention", "latent_attention")


@dataclass(frozen=True)
class KerepelLayer:
    type: str
    mixer: Any              # AttentionSizes or LatentAttentionSizes
    mlp: Any                # DenseSizes, MoeSizes, or None: the layer has no feed-forward

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


@dataclass(frozen=True)
class KerepelConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[KerepelLayer, ...]
    bigram: PairTable | None = None
    side_dim: int = 0               # token_side.dim; 0: no per-layer token input
    logit_scale: float | None = None    # None: config.json gives none, the logits stay as they are
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(raw: dict[str, Any]) -> "KerepelConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json is missing the 'norm' entry with its eps")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        layers: list[KerepelLayer] = []
        for index, entry in enumerate(entries):
            where = f"layers[{index}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where} has type {kind!r}; known: {', '.join(MIXER_TYPES)}")
            if not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs the sizes of its mixer")
            if kind == "attention":
                mixer = AttentionSizes.from_dict(entry["mixer"], where + ".mixer")
                if mixer.kv_from is not None:
                    source = layers[mixer.kv_from] if mixer.kv_from < index else None
                    if source is None or source.type != "attention" or source.mixer.kv_from is not None:
                        raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier attention layer with keys of its own")
                    theirs, mine = source.mixer, mixer
                    if (theirs.kv_heads, theirs.dim, theirs.vdim) != (mine.kv_heads, mine.dim, mine.vdim):
                        raise ConfigError(f"config.json: {where} reads the keys of layer {mixer.kv_from}, whose key/value heads differ")
            else:
                mixer = LatentAttentionSizes.from_dict(entry["mixer"], where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is None:
                feed = None
            elif isinstance(mlp, dict) and mlp.get("kind") == "dense":
                feed = DenseSizes(_int(mlp, "ff", where + ".mlp"))
            elif isinstance(mlp, dict) and mlp.get("kind") == "moe":
                feed = MoeSizes.from_dict(mlp, where + ".mlp")
            else:
                raise ConfigError(f"config.json: {where}.mlp must be null or of kind 'dense' or 'moe'")
            layers.append(KerepelLayer(kind, mixer, feed))
        pair = (raw.get("embedding") or {}).get("bigram")
        bigram = None
        if pair:
            bigram = PairTable(_int(pair, "buckets", "embedding.bigram"), _int(pair, "mul_prev", "embedding.bigram", 0),
                               _int(pair, "mul_cur", "embedding.bigram", 0))
        side = raw.get("token_side") or {}
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return KerepelConfig(_int(raw, "vocab", "the model"), _int(raw, "width", "the model"), _float(norm, "eps", "norm"), tuple(layers),
                             bigram, _int(side, "dim", "token_side") if side else 0,
                             _float(raw, "logit_scale", "the model") if raw.get("logit_scale") is not None else None, eos_ids)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture}
        if self.bigram is not None:
            out["embedding"] = {"bigram": self.bigram.to_dict()}
        out["layers"] = [layer.to_dict() for layer in self.layers]
        if self.logit_scale is not None:
            out["logit_scale"] = self.logit_scale
        out["norm"] = {"eps": self.eps}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        out.update({"vocab": self.vocab, "width": self.width})
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
