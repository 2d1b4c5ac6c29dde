from .base import (Block, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, ResidualStream,
                   StepContext, block_class, build_part, register_block, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position, unregister)
from . import attention, block, embedding, mlp, rmsnorm, rope  # noqa: F401  (registers the built-in kinds)
from .attention import AttentionMixer
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .mlp import GatedMLP
from .rmsnorm import RMSNorm
from .rope import RotaryPosition

__all__ = ["Block", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding", "ResidualStream",
           "StepContext", "block_class", "build_part", "register_block", "register_embedding",
           "register_feed_forward", "register_head", "register_mixer", "register_norm", "register_position", "unregister", "AttentionMixer", "PreNormBlock", "OutputHead",
           "TokenEmbedding", "GatedMLP", "RMSNorm", "RotaryPosition"]
