from . import attention, block, conv_attention, ends, latent_attention, lightning, mlp, norm, pair, pass_input, recurrent, rope, routed_experts, token_input    # register the built-in kinds
from .base import (CacheRequest, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Rotation, lookup,
                   register_block, register_embedding, register_feed_forward, register_head, register_mixer, register_norm,
                   register_position)
from .linear import Linear
from .pass_input import PassInput, register_pass_input
from .runtime import Runtime
from .token_input import TokenInput, register_token_input
