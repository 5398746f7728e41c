from .base import Block, FeedForward, Mixer, Norm, PositionEncoding, Runtime
from .registry import build_part, register_part, registered_parts, unregister_part
from .spec import (ActMLPSpec, AttentionSpec, BiasedAttentionSpec, BigramEmbeddingSpec, ChannelDecaySpec, ChannelDeltaSpec, ConvInputSpec,
                   DeltaRuleSpec, DepthAverageSpec, RotNormAttentionSpec,
                   DiffAttentionSpec, GLASpec, LatentAttentionSpec, LayerSpec, LoopSpec, Mamba2Spec, MLSTMSpec, ModelSpec, MoESpec,
                   PositionedEmbeddingSpec, RMSNormSpec, RotarySpec, SideBySideSpec, SwiGLUSpec, TableMoESpec, TanhNormSpec, YarnScaling)
from . import (attention, bias_attention, block, channel_recurrent, conv_input, depth_average, diff_attention, embedding,   # registers the
               latent_attention, loop, mlp, moe, recurrent, rmsnorm, rot_norm_attention, rotary, side_by_side, tanh_norm)  # built-in parts
from .linear import Linear
