from .block import HyperConnectionBlock, PreNormBlock, SublayerNormBlock
from .context import StepContext, Workspace
from .embedding import LMHead, TokenEmbedding
from .feed_forward import DenseMLP, GatedMLP
from .latent_attention import LatentAttention
from .mingru import MinGRUMixer
from .mixer import CausalSelfAttention
from .moe import RoutedExperts
from .norm import GroupRMSNorm, LayerNorm, ShiftedRMSNorm, StreamSumRMSNorm
from .parallel import ParallelMixer
from .position import LearnedAbsolutePositions, RotaryPositions
from .state_space import StateSpaceMixer
from .window_attention import WindowAttention
from .registry import get_part, part_names, register_part, unregister_part

__all__ = ["MinGRUMixer", "ShiftedRMSNorm", "HyperConnectionBlock", "GatedMLP", "StreamSumRMSNorm", "ParallelMixer", "StateSpaceMixer", "WindowAttention", "PreNormBlock", "SublayerNormBlock", "LatentAttention", "RoutedExperts", "GroupRMSNorm", "RotaryPositions", "StepContext", "Workspace", "LMHead", "TokenEmbedding", "DenseMLP",
           "CausalSelfAttention", "LayerNorm", "LearnedAbsolutePositions", "get_part", "part_names",
           "register_part", "unregister_part"]
