"""The parts a model is assembled from.  Importing the package registers the built-in
kinds; a new kind is added by decorating a class with the registry of its role."""
from . import arrangement, attention, attention_forms, depth, embedding, ffn, latent_attention, moe, norm, recurrent, rope, shift, side  # noqa: F401  (registration)
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, REGISTRIES, SHIFTS, SIDES, Arrangement, Delta,
                   Embedding, FeedForward, Head, InputShift, KVNeed, Mixer, Norm, Part, PositionEncoding, SideInput, StateNeed, WeightDecl)
from .linear import GatedLinear, Linear
from .spec import LayerSpec, ModelSpec, PartSpec, Run

__all__ = [
    "ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "REGISTRIES", "SHIFTS", "SIDES", "InputShift", "SideInput",
    "Arrangement", "Delta", "Embedding", "FeedForward", "Head", "KVNeed", "Mixer", "Norm", "Part", "PositionEncoding",
    "StateNeed", "WeightDecl", "GatedLinear", "Linear", "LayerSpec", "ModelSpec", "PartSpec", "Run",
]
