from . import attention, attention_kv, block, delta_rule, embedding, mlp, norm, polynorm, rope, short_conv  # noqa: F401  (registers the built-in parts)
from .base import (BLOCKS, CONVOLUTIONS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheNeed, Embedding,
                   FeedForward, Head, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec, PositionEncoding, Registry, RotaryTable,
                   RunMemory, RunSpec, Runtime, ShortConvolution, StateNeed, StepContext, TensorSpec)

__all__ = [
    "BLOCKS", "CONVOLUTIONS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheNeed", "Embedding",
    "FeedForward", "Head", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec", "PositionEncoding", "Registry",
    "RotaryTable", "RunMemory", "RunSpec", "Runtime", "ShortConvolution", "StateNeed", "StepContext", "TensorSpec",
]
