"""Parts a layer is put together from: norm, position encoding, mixer, feed-forward, block."""

from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, FeedForward, Mixer, Norm,
                   Part, PositionEncoding, Runtime)
from .norm import RMSNorm
from .rotary import Rotary
from .attention import GQAAttention
from .mlp import GatedMLP
from .block import PreNormBlock

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Block", "FeedForward", "Mixer",
           "Norm", "Part", "PositionEncoding", "Runtime", "RMSNorm", "Rotary", "GQAAttention",
           "GatedMLP", "PreNormBlock"]
