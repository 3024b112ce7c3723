"""Parts a layer is put together from; registered by kind."""
from ..registry import register_part
from .base import (FeedForward, KvCacheSpec, Mixer, Norm, Part, PositionEncoding, StateSpec,
                   TensorDecl)
from .linear import Linear
from .norm import LayerNorm, RmsNorm, ScalarRmsNorm
from .rope import RopeInterleaved, RopeNeox
from .mlp import GluMlp, Relu2Mlp, SwiGluMlp
from .attention import GqaAttention
from .hgrn2 import Hgrn2Mixer
from .diff_attention import DiffAttention
from .moe import GroupedMoe, MoeSwiGlu, ScoredMoe
from .latent_attention import LatentAttention
from .normed_attention import NormedAttention
from .rglru import RgLruMixer
from .ssd import SsdMixer
from .parallel import ParallelMixer
from .block import GatedPostNormBlock, HyperPreNormBlock, PreNormBlock

register_part("norm", "rmsnorm", RmsNorm)
register_part("position", "rope_neox", RopeNeox)
register_part("feed_forward", "swiglu", SwiGluMlp)
register_part("mixer", "gqa_attention", GqaAttention)
register_part("block", "prenorm", PreNormBlock)
register_part("norm", "rmsnorm_scalar", ScalarRmsNorm)
register_part("position", "rope_interleaved", RopeInterleaved)
register_part("mixer", "hgrn2", Hgrn2Mixer)
register_part("mixer", "diff_attention", DiffAttention)
register_part("feed_forward", "moe_swiglu", MoeSwiGlu)
register_part("block", "gated_postnorm", GatedPostNormBlock)
register_part("norm", "layernorm", LayerNorm)
register_part("mixer", "latent_attention", LatentAttention)
register_part("feed_forward", "relu2", Relu2Mlp)
register_part("feed_forward", "glu", GluMlp)
register_part("feed_forward", "moe_grouped", GroupedMoe)
register_part("block", "hyper_prenorm", HyperPreNormBlock)
register_part("mixer", "normed_attention", NormedAttention)
register_part("mixer", "rglru", RgLruMixer)
register_part("mixer", "parallel", ParallelMixer)
register_part("mixer", "ssd", SsdMixer)
register_part("feed_forward", "moe_scored", ScoredMoe)

__all__ = ["FeedForward", "KvCacheSpec", "Mixer", "Norm", "Part", "PositionEncoding", "StateSpec",
           "TensorDecl", "Linear", "RmsNorm", "ScalarRmsNorm", "RopeNeox", "RopeInterleaved", "SwiGluMlp", "GqaAttention",
           "Hgrn2Mixer", "DiffAttention", "MoeSwiGlu", "PreNormBlock", "GatedPostNormBlock", "LayerNorm", "GluMlp", "Relu2Mlp",
           "GroupedMoe", "LatentAttention", "HyperPreNormBlock", "NormedAttention", "RgLruMixer", "ParallelMixer", "SsdMixer", "ScoredMoe"]
