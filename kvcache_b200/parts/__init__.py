from .attention import GQAAttention
from .base import (Block, FeedForward, LayerContext, Mixer, Norm, PagedKVSpec, PagedKVView, Part,
                   PositionEncoding, Rotation, StateSpec, StepBatch, StepPlan, StepPlanner, TORCH_DTYPES)
from .block import PreNormBlock, ResidualGate, SandwichBlock
from .feedforward import GatedMLP, ReluSquaredMLP, RoutedMLP
from .token_shift import TokenShiftMixer
from .latent_attention import LatentAttention
from .stream import LoopEntry
from .model import CacheEntry, DecoderModel, LayerCall
from .norm import RMSNorm
from .position import NoPositionEncoding, RampScaling, RotaryHalf

__all__ = ["GQAAttention", "Block", "FeedForward", "LayerContext", "Mixer", "Norm", "PagedKVSpec",
           "PagedKVView", "Part", "PositionEncoding", "Rotation", "StateSpec", "StepBatch", "StepPlan", "StepPlanner", "TORCH_DTYPES",
           "PreNormBlock", "GatedMLP", "CacheEntry", "DecoderModel", "LayerCall", "RMSNorm",
           "NoPositionEncoding", "RotaryHalf", "RampScaling", "SandwichBlock", "RoutedMLP", "LatentAttention", "LoopEntry",
           "ResidualGate", "ReluSquaredMLP", "TokenShiftMixer"]
