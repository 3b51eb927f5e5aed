from .base import (Block, DeferredNorm, FeedForward, InputStage, LayerCache, Mixer, Norm, OutputStage, PagedCacheSpec, Part,
                   PendingSum, PositionEncoding, StateSpec, StreamStage, WeightSpec, known_parts, part_class,
                   register_part, settle)
from .norm import LayerNorm, RMSNorm
from .rotary import RotaryEncoding, rotary_frequencies, yarn_attention_factor, yarn_frequencies
from .attention import GQAAttention, SinkGQAAttention, distance_slopes
from .mlp import GatedMLP, SwiGLU
from .moe import RoutedExperts
from .latent_attention import LatentAttention
from .delta_rule import GatedDeltaMixer
from .ssm import SelectiveStateMixer
from .embedding import LearnedPositions, NormedHead, OutputHead, TokenEmbedding
from .block import ParallelBlock, PostNormBlock, PreNormBlock
from .stream import StreamInputMix
from .plan import ModelPlan, Run

__all__ = ["Block", "DeferredNorm", "FeedForward", "InputStage", "OutputStage", "NormedHead", "LayerCache", "Mixer", "Norm", "PagedCacheSpec", "Part",
           "PositionEncoding", "StateSpec", "WeightSpec", "known_parts", "part_class",
           "register_part", "RMSNorm", "RotaryEncoding", "rotary_frequencies", "GQAAttention",
           "SwiGLU", "OutputHead", "TokenEmbedding", "PreNormBlock", "ModelPlan", "Run",
           "GatedMLP", "RoutedExperts", "LatentAttention", "GatedDeltaMixer", "PostNormBlock",
           "yarn_frequencies", "yarn_attention_factor", "PendingSum", "StreamStage", "settle", "LayerNorm",
           "SinkGQAAttention", "distance_slopes", "LearnedPositions", "ParallelBlock", "StreamInputMix",
           "SelectiveStateMixer"]
