"""Parts of a layer.  Importing this package registers the built-in kinds."""

from .base import Block, FeedForward, Mixer, Norm, ParamSpec, Part
from .norm import LayerNorm, RMSNorm
from .rope import RotaryEncoding, RotaryPairs, ScaledRotary, pair_frequencies, rope_tables, scaled_frequencies
from .attention import AttentionMixer
from .latent_attention import LatentAttentionMixer
from .gla import GatedLinearAttentionMixer
from .lightning import LightningMixer
from .gated_delta import GatedDeltaMixer
from .general_delta import GeneralDeltaMixer
from .side_by_side import SideBySideMixer
from .swiglu import SwiGLU, join_gate_up
from .moe import RoutedFeedForward
from .block import ParallelBlock, PreNormBlock, SandwichBlock, SublayerNormBlock

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part", "RMSNorm", "RotaryEncoding",
           "rope_tables", "AttentionMixer", "SwiGLU", "join_gate_up", "PreNormBlock", "LayerNorm", "ScaledRotary",
           "scaled_frequencies", "LatentAttentionMixer", "GatedLinearAttentionMixer", "RoutedFeedForward",
           "SublayerNormBlock", "ParallelBlock", "RotaryPairs", "pair_frequencies", "LightningMixer", "GatedDeltaMixer",
           "SideBySideMixer", "GeneralDeltaMixer", "SandwichBlock"]
