from .base import (Block, CompositeRequest, FeedForward, KeyValueRequest, LayerSpec, Mixer, ModelPlan, Norm,
                   Part, PartSpec, PositionEncoding, ScheduleEntry, StateRequest)
from .linear import LinearWeight
from .norm import RMSNorm
from .rope import DistancePenalty, RotaryEmbedding
from .attention import Attention
from .mlp import GatedMLP
from .recurrent import GatedDeltaRule, Retention
from .parallel import ParallelMixer
from .moe import MixtureOfExperts
from .block import PreNormBlock, PreNormMixerBlock

__all__ = ["Block", "CompositeRequest", "FeedForward", "KeyValueRequest", "LayerSpec", "Mixer", "ModelPlan", "Norm",
           "Part", "PartSpec", "PositionEncoding", "ScheduleEntry", "StateRequest", "LinearWeight",
           "RMSNorm", "RotaryEmbedding", "DistancePenalty", "Attention", "GatedMLP", "Retention", "GatedDeltaRule",
           "ParallelMixer", "MixtureOfExperts", "PreNormBlock", "PreNormMixerBlock"]
