"""Parts of a decoder layer: mixers, feed-forwards, norms, position encodings, blocks."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward, KVRequest, Mixer,
                   Norm, Part, PositionEncoding, Registry, RotaryParams, StateRequest, WeightSpec, walk_parts)
from .attention import GqaAttention
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .feedforward import SwiGLU
from .linear import linear
from .norm import RMSNorm
from .rope import RotaryEncoding
from .shortconv import ShortConv
