from .attention import Attention
from .convattn import ConvNormAttention
from .base import (FeedForward, Mixer, Norm, Part, PendingLinear, PendingNorm, PositionEncoding, Runtime, ScaledRows,
                   StepContext)
from .block import ConvPreNormBlock, ParallelBlock, PostNormBlock, PreNormBlock, SandwichBlock, TokenConv, TokenShift
from .embedding import BigramEmbedding, Embedding, OutputHead
from .linear import JoinedLinear, Linear
from .latent import LatentAttention
from .mlp import CappedGLU, GeluGLU, MixtureOfExperts, SwiGLU
from .norm import LayerNorm, RMSNorm
from .parallel import NormedParallelMixers, ParallelMixers
from .recurrent import MLSTM, MinGRU, Retention
from .rope import FrequencyRamp, NoPosition, RotaryHalf, RotaryPairs, rotary_inv_freq
from .scored import ScoredAttention

__all__ = ["Attention", "FeedForward", "Mixer", "Norm", "Part", "PendingLinear", "PendingNorm", "ScaledRows", "PositionEncoding", "Runtime",
           "StepContext", "PreNormBlock", "ConvPreNormBlock", "TokenConv", "Embedding", "OutputHead", "Linear", "JoinedLinear",
           "SwiGLU", "CappedGLU", "RMSNorm", "ParallelMixers", "MinGRU", "Retention", "NoPosition", "RotaryHalf",
           "rotary_inv_freq", "ParallelBlock", "LatentAttention", "MixtureOfExperts", "MLSTM", "RotaryPairs", "FrequencyRamp", "ScoredAttention", "LayerNorm", "SandwichBlock", "TokenShift",
           "PostNormBlock", "BigramEmbedding", "GeluGLU", "NormedParallelMixers", "ConvNormAttention"]
