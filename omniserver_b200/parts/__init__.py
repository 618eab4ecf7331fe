"""Parts a decoder is put together from, chosen by name through registries."""

from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, CacheBinding, FeedForward, KVCacheNeed,
                   Mixer, Norm, ParamSpec, Part, PartSpec, PositionEncoding, RotaryOperands, StateNeed, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position_encoding)
from . import blocks, embedding, feedforward, mixers, norms, positions  # noqa: F401  (fill the registries)
from .blocks import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .feedforward import SwiGLU
from .linear import Linear
from .mixers import GQAAttention
from .norms import RMSNorm
from .positions import MRope, ROPE_STATE
