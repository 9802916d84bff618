from . import standard  # registers the standard parts
from . import dynamic_tanh, delta_rule, latent_attention, routed  # noqa: F401  (more parts)
from . import rms_norm, biased_attention, lightning, paired  # noqa: F401
from . import pooled_attention, rglru  # noqa: F401
from . import retention, span_attention, time_mix, token_side  # noqa: F401
from .base import (CacheRequest, Embedding, FeedForward, Head, Mixer, Norm, Part,
                   PositionEncoding, TensorRequest, build_part, register_embedding,
                   register_feed_forward, register_head, register_mixer, register_norm,
                   register_position, registered)
from .model import (Block, CacheGroup, Model, OutputNormBlock, ParallelBlock, PreNormBlock,
                    SandwichNormBlock, register_arrangement)
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

__all__ = [
    "Block", "CacheGroup", "CacheRequest", "Embedding", "FeedForward", "Head", "LayerCall",
    "LayerSpec", "Mixer", "Model", "ModelSpec", "Norm", "OutputNormBlock", "Part", "PartSpec", "PositionEncoding",
    "ParallelBlock", "PreNormBlock", "SandwichNormBlock", "TensorRequest", "build_part", "register_arrangement",
    "register_embedding", "register_feed_forward", "register_head", "register_mixer",
    "register_norm", "register_position", "registered",
]
