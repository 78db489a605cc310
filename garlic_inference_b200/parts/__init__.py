"""Parts a model is put together from; importing this package registers the built-in ones."""
from .base import (Block, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Runtime,
                   StepContext, StepShape, known_parts, part_class, register_part)
from .attention import GQAAttention
from .block import LinearHead, PreNormResidualBlock, TokenEmbedding
from .mlp import SwiGLUMLP
from .norm import RMSNorm
from .rotary import RotaryPositions

__all__ = ["Block", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding",
           "Runtime", "StepContext", "StepShape", "known_parts", "part_class", "register_part", "GQAAttention",
           "LinearHead", "PreNormResidualBlock", "TokenEmbedding", "SwiGLUMLP", "RMSNorm", "RotaryPositions"]
