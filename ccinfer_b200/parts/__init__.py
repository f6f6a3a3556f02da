from .attention import GroupedQueryAttention
from .base import (Block, CachedTensor, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, Residual, StateNeed,
                   TensorSpec)
from .block import LayerScaleBlock, PostNormBlock, PreNormBlock, SandwichNormBlock
from .delta import ChannelGatedDelta
from .embedding import LoopInput, OutputHead, TokenEmbedding, TokenSideInput
from .feedforward import ClampedGLU, SquaredReLU, SwiGLU
from .latent import LatentAttention
from .linear_attention import GatedLinearAttention
from .moe import MixtureOfExperts
from .norm import RMSNorm, StreamRows
from .parallel import ParallelMixers
from .position import NoPosition, QueryTemperature, RotaryHalf
from .ssm import SelectiveStateSpace

__all__ = ["Block", "CachedTensor", "CacheNeed", "ChannelGatedDelta", "ClampedGLU", "FeedForward",
           "GatedLinearAttention", "GroupedQueryAttention", "LatentAttention", "LayerScaleBlock", "LoopInput", "Mixer",
           "MixtureOfExperts", "NoPosition", "Norm", "OutputHead", "ParallelMixers", "Part", "PositionEncoding",
           "PostNormBlock", "PreNormBlock", "QueryTemperature", "RMSNorm", "Residual", "RotaryHalf", "SandwichNormBlock", "SelectiveStateSpace",
           "SquaredReLU", "StateNeed", "StreamRows", "SwiGLU", "TensorSpec", "TokenEmbedding", "TokenSideInput"]
