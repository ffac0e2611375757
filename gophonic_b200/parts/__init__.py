"""The parts a decoder is assembled from, and their registration under their kind names."""
from .. import registry
from .base import (FeedForward, KVRequest, Mixer, Norm, Part, PositionEncoding, Runtime, StateRequest,
                   TensorDecl)
from .attention import Attention
from .block import PreNormBlock
from .norm import RMSNorm
from .rope import NoPosition, RotaryEmbedding
from .swiglu import SwiGLU

registry.register_norm("rmsnorm", RMSNorm)
registry.register_position("rope", RotaryEmbedding)
registry.register_position("none", NoPosition)
registry.register_mixer("attention", Attention)
registry.register_feed_forward("swiglu", SwiGLU)
registry.register_block("prenorm", PreNormBlock)

__all__ = ["Attention", "FeedForward", "KVRequest", "Mixer", "NoPosition", "Norm", "Part", "PositionEncoding",
           "PreNormBlock", "RMSNorm", "RotaryEmbedding", "Runtime", "StateRequest", "SwiGLU", "TensorDecl"]
