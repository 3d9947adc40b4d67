from .base import (Block, FeedForward, KeyValueRequest, LayerSpec, Mixer, ModelPlan, Norm, Part,
                   PartSpec, PositionEncoding, ScheduleEntry, StateRequest)
from .linear import LinearWeight
from .norm import RMSNorm
from .rope import RotaryEmbedding
from .attention import Attention
from .mlp import GatedMLP
from .block import PreNormBlock

__all__ = ["Block", "FeedForward", "KeyValueRequest", "LayerSpec", "Mixer", "ModelPlan", "Norm",
           "Part", "PartSpec", "PositionEncoding", "ScheduleEntry", "StateRequest", "LinearWeight",
           "RMSNorm", "RotaryEmbedding", "Attention", "GatedMLP", "PreNormBlock"]
