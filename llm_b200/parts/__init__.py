from . import spec
from .base import (Block, FeedForward, Mixer, Norm, Part, PositionEncoding, StepContext,
                   build_block, build_feed_forward, build_mixer, build_norm, build_position,
                   register_block, register_feed_forward, register_mixer, register_norm,
                   register_position)
from .attention import AttentionMixer
from .block import ParallelBlock, PreNormBlock, SandwichBlock
from .delta_rule import DeltaRuleMixer
from .diff_attention import DiffAttentionMixer
from .feedforward import GatedMlp, Mlp
from .gated_attention import GatedAttentionMixer
from .gated_recurrence import GatedRecurrenceMixer
from .latent_attention import LatentAttentionMixer
from .norm import RmsNorm, TanhNorm
from .projected import ProjectedMixer
from .routed_experts import RoutedExperts
from .side_by_side import SideBySideMixer
from .sigmoid_attention import SigmoidAttentionMixer
from .state_space import StateSpaceMixer
from .position import Rope, inverse_frequencies

__all__ = ["spec", "Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
           "StepContext", "build_block", "build_feed_forward", "build_mixer", "build_norm",
           "build_position", "register_block", "register_feed_forward", "register_mixer",
           "register_norm", "register_position", "AttentionMixer", "DiffAttentionMixer", "ParallelBlock", "PreNormBlock", "GatedMlp",
           "RmsNorm", "Rope", "inverse_frequencies", "TanhNorm", "ProjectedMixer", "LatentAttentionMixer",
           "SigmoidAttentionMixer", "GatedRecurrenceMixer", "SideBySideMixer", "SandwichBlock", "DeltaRuleMixer",
           "GatedAttentionMixer", "Mlp", "RoutedExperts", "StateSpaceMixer"]
