from .base import (Block, Embedding, FeedForward, Head, HostStep, Mixer, Norm, ParamSpec, Part, Piece, PositionEncoding,
                   StepWork, whole)
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .feedforward import SwiGLUFeedForward
from .mixer import AttentionMixer
from .norm import RMSNorm
from .position import RotaryEncoding
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, make, register_block,
                       register_feed_forward, register_mixer, register_norm, register_position_encoding)

register_mixer("attention")(AttentionMixer)
register_feed_forward("swiglu")(SwiGLUFeedForward)
register_norm("rmsnorm")(RMSNorm)
register_position_encoding("rotary")(RotaryEncoding)
register_block("pre_norm")(PreNormBlock)
