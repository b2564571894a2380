from . import (attention, attention_kv, block, delta_rule, embedding, latent_attention, linear_recurrence, mlp, moe, norm, polynorm, reentry, rope,  # noqa: F401
               short_conv, side_by_side, talking_attention)      # (importing registers the built-in parts)
from .base import (BLOCKS, CONVOLUTIONS, EMBEDDINGS, FEED_FORWARDS, HEADS, JUNCTIONS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheNeed, Embedding,
                   FeedForward, Head, Junction, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec, PositionEncoding, Registry, RotaryTable,
                   RunMemory, RunSpec, Runtime, ShortConvolution, StateNeed, StepContext, TensorSpec)

__all__ = [
    "BLOCKS", "CONVOLUTIONS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "JUNCTIONS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheNeed", "Embedding",
    "FeedForward", "Head", "Junction", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec", "PositionEncoding", "Registry",
    "RotaryTable", "RunMemory", "RunSpec", "Runtime", "ShortConvolution", "StateNeed", "StepContext", "TensorSpec",
]
