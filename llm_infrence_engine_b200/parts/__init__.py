from .attention import PagedAttention
from .base import (INIT_NORM, INIT_NORMAL, MATRIX, TABLE, VECTOR, FeedForward, Mixer, Norm, ParamSpec, Part,
                   PositionEncoding, Source, walk)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .mlp import GatedMLP
from .norm import RMSNorm
from .rotary import RotaryEncoding

__all__ = ["PagedAttention", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part", "PositionEncoding", "Source", "walk",
           "PreNormBlock", "OutputHead", "TokenEmbedding", "GatedMLP", "RMSNorm", "RotaryEncoding",
           "INIT_NORM", "INIT_NORMAL", "MATRIX", "TABLE", "VECTOR"]
