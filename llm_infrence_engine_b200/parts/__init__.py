from .attention import PagedAttention
from .attention_biased import BiasedAttention
from .attention_latent import LatentAttention
from .attention_masked import MaskedAttention
from .base import (ANY, INIT_EYE, INIT_NORM, INIT_NORMAL, INIT_ONES, INIT_SHARE, INIT_SMALL, MATRIX, TABLE, VECTOR, FeedForward, Mixer, Norm, ParamSpec, Part,
                   PositionEncoding, Source, walk)
from .block import ParallelBlock, PreNormBlock, SandwichBlock
from .embedding import OutputHead, TokenEmbedding
from .hyper import HyperConnection, HyperConnectionBlock, ResidualStreams
from .mlp import ClampedGLU, DenseMLP, GatedMLP, GatedUnit, RoutedExperts
from .norm import LayerNorm, RMSNorm
from .recurrent import GatedDeltaMixer, HeadDecayDeltaMixer, MatrixMemoryMixer, ParallelMixer, SelectiveScanMixer, StateSpaceMixer
from .rotary import RampedRotary, RotaryEncoding

__all__ = ["MatrixMemoryMixer", "MaskedAttention", "SandwichBlock", "ParallelBlock", "GatedUnit", "RoutedExperts", "HeadDecayDeltaMixer", "SelectiveScanMixer", "ClampedGLU", "LayerNorm", "GatedDeltaMixer", "ParallelMixer", "StateSpaceMixer", "RampedRotary",
           "PagedAttention", "BiasedAttention", "LatentAttention", "HyperConnection", "HyperConnectionBlock", "ResidualStreams", "DenseMLP", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part", "PositionEncoding", "Source", "walk",
           "PreNormBlock", "OutputHead", "TokenEmbedding", "GatedMLP", "RMSNorm", "RotaryEncoding",
           "ANY", "INIT_EYE", "INIT_NORM", "INIT_NORMAL", "INIT_ONES", "INIT_SHARE", "INIT_SMALL", "MATRIX", "TABLE", "VECTOR"]
