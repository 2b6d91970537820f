"""The parts a decoder is assembled from, and their registration under their kind names."""
from .. import registry
from .base import (FeedForward, KVRequest, Mixer, Norm, Part, PositionEncoding, Runtime, StateRequest,
                   TensorDecl)
from .attention import Attention
from .block import PreNormBlock
from .gated_attention import GatedAttention
from .linear_state import DecayState, MatrixMemory
from .norm import RMSNorm
from .rope import NoPosition, PairRotaryEmbedding, RotaryEmbedding
from .swiglu import SwiGLU

registry.register_norm("rmsnorm", RMSNorm)
registry.register_position("rope", RotaryEmbedding)
registry.register_position("rope_pairs", PairRotaryEmbedding)
registry.register_position("none", NoPosition)
registry.register_mixer("attention", Attention)
registry.register_mixer("gated_attention", GatedAttention)
registry.register_mixer("gla", DecayState)
registry.register_mixer("mlstm", MatrixMemory)
registry.register_feed_forward("swiglu", SwiGLU)
registry.register_block("prenorm", PreNormBlock)

__all__ = ["Attention", "DecayState", "FeedForward", "GatedAttention", "MatrixMemory", "PairRotaryEmbedding", "KVRequest", "Mixer", "NoPosition", "Norm", "Part", "PositionEncoding",
           "PreNormBlock", "RMSNorm", "RotaryEmbedding", "Runtime", "StateRequest", "SwiGLU", "TensorDecl"]
