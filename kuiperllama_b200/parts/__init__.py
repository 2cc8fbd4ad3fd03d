"""Parts of a layer: norm, position encoding, mixer, feed-forward and their arrangement."""
from .base import (FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime, StepContext, part_class,
                   register_arrangement, register_feed_forward, register_mixer, register_norm, register_position)
from .linear import Linear
from .norm import LayerNorm, NoNorm, RMSNorm
from .position import RotaryPosition, rotary_inverse_frequencies
from .attention import AttentionMixer
from .swiglu import SwiGLUFeedForward
from .block import PreNormBlock, SandwichBlock
from .dense import DenseFeedForward
from .gate import SigmoidLinearGate
from .recurrent import GatedDeltaMixer, MinGRUMixer, RGLRUMixer
from .latent_attention import LatentAttentionMixer
from .moe import MoEFeedForward
from .block import ParallelBlock
from .composite import BranchMixer, InputConvMixer, ParallelMixer
from .matrix_recurrent import GatedLinearAttentionMixer, Mamba2Mixer
from .mixed_attention import MixedHeadAttentionMixer
from .window_attention import WindowAttentionMixer

__all__ = ["FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "StepContext", "part_class",
           "register_arrangement", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "Linear", "RMSNorm", "RotaryPosition", "rotary_inverse_frequencies",
           "AttentionMixer", "SwiGLUFeedForward", "PreNormBlock", "SandwichBlock", "LayerNorm", "DenseFeedForward",
           "SigmoidLinearGate", "GatedDeltaMixer", "MinGRUMixer", "RGLRUMixer", "LatentAttentionMixer", "MoEFeedForward", "ParallelBlock", "BranchMixer", "InputConvMixer",
           "ParallelMixer", "GatedLinearAttentionMixer", "Mamba2Mixer", "MixedHeadAttentionMixer", "WindowAttentionMixer"]
