from .attention import Attention, AttentionSpec
from .base import Block, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, StateNeed, WeightDecl
from .block import OutputNormBlock, OutputNormBlockSpec, PreNormBlock, PreNormBlockSpec, SandwichBlock, SandwichBlockSpec
from .delta_rule import GatedDeltaRule, GatedDeltaRuleSpec
from .latent_attention import LatentAttention, LatentAttentionSpec
from .lightning import ConstantDecayAttention, ConstantDecayAttentionSpec
from .linear_attention import GatedLinearAttention, GatedLinearAttentionSpec
from .mamba2 import Mamba2, Mamba2Spec
from .mlstm import MatrixLstm, MatrixLstmSpec
from .moe import RoutedExperts, RoutedExpertsSpec
from .mlp import GatedMlp, GatedMlpSpec
from .model import DecoderModel, ResidualStream, declared_weights
from .norm import DynTanh, DynTanhSpec, RmsNorm, RmsNormSpec
from .parallel import ParallelBlock, ParallelBlockSpec, ParallelMixer, ParallelMixerSpec
from .rglru import RgLru, RgLruSpec
from .registry import build_model, build_part, register_model, register_part, registered_models, registered_parts
from .rotary import Rotary, RotarySpec

__all__ = ["Attention", "AttentionSpec", "Block", "CacheNeed", "FeedForward", "Mixer", "Norm", "Part",
           "PositionEncoding", "StateNeed", "WeightDecl", "PreNormBlock", "PreNormBlockSpec", "OutputNormBlock", "OutputNormBlockSpec", "GatedDeltaRule", "GatedDeltaRuleSpec", "RgLru", "RgLruSpec", "GatedMlp",
           "GatedMlpSpec", "GatedLinearAttention", "GatedLinearAttentionSpec", "ParallelBlock", "ParallelBlockSpec",
           "ParallelMixer", "ParallelMixerSpec", "LatentAttention", "LatentAttentionSpec", "Mamba2", "Mamba2Spec", "MatrixLstm",
           "MatrixLstmSpec", "RoutedExperts", "RoutedExpertsSpec", "DynTanh", "DynTanhSpec", "DecoderModel", "ResidualStream", "declared_weights", "RmsNorm", "RmsNormSpec",
           "SandwichBlock", "SandwichBlockSpec", "ConstantDecayAttention", "ConstantDecayAttentionSpec",
           "build_model", "build_part", "register_model", "register_part", "registered_models", "registered_parts", "Rotary", "RotarySpec"]
