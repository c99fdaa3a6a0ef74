"""Model parts: plan data, interfaces, registries and the built-in parts."""

from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry, sequential_order
from .base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
    Block, BuildEnv, DeferredLinear, Embedding, FeedForward, FixedState, Head, Mixer, Norm, PagedKV,
    Part, PositionEncoding, Registry, Stream,
)
from . import norm, position, attention, short_conv, feed_forward, block, embedding  # register built-ins
from .model import Model

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "Block", "BuildEnv", "DeferredLinear", "Embedding", "FeedForward", "FixedState", "Head", "LayerSpec", "Mixer",
    "Model", "ModelPlan", "Norm", "PagedKV", "Part", "PartSpec", "PositionEncoding", "Registry",
    "RunEntry", "Stream", "sequential_order",
]
