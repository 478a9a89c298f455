from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildEnv,
                   FeedForward, Mixer, Norm, Part, PositionEncoding, Projected, build_part, register_block, register_embedding,
                   register_feed_forward, register_head, register_mixer, register_norm, register_position_encoding)
from .context import GroupContext, KVCacheView, StateCacheView, StepContext, Workspace
from . import (attention, block, delta_rule, embedding, experts, gated_linear_attention, latent_attention, linear_attention, mlp, norm, pair,  # noqa: F401
               recurrent, rope, sigmoid_attention, sink_attention, window_attention)  # noqa: F401  (register the built-in parts)
from .model import DecoderModel, expected_tensors

__all__ = [n for n in dir() if not n.startswith("_")]
