"""Registers the built-in parts."""
from .attention import AttentionMixer
from .base import register_part
from .block import ParallelResidualBlock, PreNormResidualBlock
from .embedding import LinearHead, TokenEmbedding
from .feedforward import DenseFeedForward, SwiGLU
from .linear_attention import DecayLinearAttention
from .norm import RMSNorm
from .position import NoPosition, RotaryInterleaved, RotaryNeox
from .shortconv import ShortConvMixer
from .sidebyside import SideBySideMixer
from .streamop import StretchEntry

register_part("mixer", "attention", AttentionMixer, replace=True)
register_part("mixer", "short_conv", ShortConvMixer, replace=True)
register_part("feed_forward", "swiglu", SwiGLU, replace=True)
register_part("norm", "rmsnorm", RMSNorm, replace=True)
register_part("position", "rope_neox", RotaryNeox, replace=True)
register_part("position", "none", NoPosition, replace=True)
register_part("block", "prenorm_residual", PreNormResidualBlock, replace=True)
register_part("embedding", "token_table", TokenEmbedding, replace=True)
register_part("head", "linear", LinearHead, replace=True)
register_part("mixer", "decay_linear_attention", DecayLinearAttention, replace=True)
register_part("mixer", "side_by_side", SideBySideMixer, replace=True)
register_part("feed_forward", "dense", DenseFeedForward, replace=True)
register_part("position", "rope_interleaved", RotaryInterleaved, replace=True)
register_part("block", "parallel_residual", ParallelResidualBlock, replace=True)
register_part("stream_op", "stretch_entry", StretchEntry, replace=True)
