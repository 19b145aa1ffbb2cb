from .attention import DifferentialAttention, GQAAttention
from .base import (KVCacheSpec, MATRIX, ParamSpec, Part, Precision, StateSpec, StepTables, TABLE, VECTOR, part_class,
                   register_part)
from .block import PostNormBlock, PreNormBlock, SandwichNormBlock
from .embedding import OutputHead, TokenEmbedding
from .feed_forward import PolyNormFeedForward, RoutedFeedForward, SwiGLUFeedForward
from .latent_attention import LatentAttention
from .norm import RMSNorm
from .parallel import ParallelMixer
from .position import RopeScaling, RotaryEmbedding
from .recurrent import GatedDeltaRule, GeneralDeltaRule, MLSTM, MinGRU, Retention, ShortConvolution
from .side_input import TokenSideInput

__all__ = [
    "DifferentialAttention", "GQAAttention", "GatedDeltaRule", "Retention", "ShortConvolution", "GeneralDeltaRule", "MLSTM", "ParallelMixer", "TokenSideInput", "KVCacheSpec", "LatentAttention", "MinGRU", "PostNormBlock", "PolyNormFeedForward", "RoutedFeedForward", "SandwichNormBlock", "MATRIX", "OutputHead", "ParamSpec", "Part", "Precision", "PreNormBlock",
    "RMSNorm", "RopeScaling", "RotaryEmbedding", "StateSpec", "StepTables", "SwiGLUFeedForward", "TABLE", "TokenEmbedding", "VECTOR",
    "part_class", "register_part",
]
