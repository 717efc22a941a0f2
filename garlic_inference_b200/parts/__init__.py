"""Parts a model is put together from; importing this package registers the built-in ones."""
from .base import (Block, Embedding, FeedForward, Gate, Head, Mixer, Norm, Part, PositionEncoding, Runtime,
                   StepContext, StepShape, StreamOffset, known_parts, part_class, register_part)
from .attention import GQAAttention
from .block import (ChannelScale, LinearHead, ParallelResidualBlock, PostNormGatedResidualBlock, PreNormResidualBlock,
                    PreNormScaledResidualBlock, SigmoidGate, StreamOffsetTable, TokenEmbedding)
from .delta_rule import GatedDeltaRule
from .latent_attention import LatentAttention
from .linear_attention import DecayLinearAttention
from .masked_attention import MaskedAttention
from .mlp import GluMLP, SwiGLUMLP, XieluMLP
from .moe import RoutedExperts
from .norm import DynamicTanhNorm, LayerNorm, RMSNorm
from .parallel import ParallelMixers
from .rglru import RGLRU
from .rotary import RotaryPositions

__all__ = ["Block", "Embedding", "FeedForward", "Gate", "Head", "PostNormGatedResidualBlock", "SigmoidGate",
           "GatedDeltaRule", "LatentAttention", "DecayLinearAttention", "XieluMLP", "Mixer", "Norm", "Part", "PositionEncoding",
           "Runtime", "StepContext", "StepShape", "known_parts", "part_class", "register_part", "GQAAttention",
           "LinearHead", "PreNormResidualBlock", "TokenEmbedding", "SwiGLUMLP", "RMSNorm", "RotaryPositions",
           "ChannelScale", "PreNormScaledResidualBlock", "MaskedAttention", "GluMLP", "RoutedExperts",
           "DynamicTanhNorm", "ParallelMixers", "ParallelResidualBlock", "LayerNorm", "RGLRU", "StreamOffset",
           "StreamOffsetTable"]
