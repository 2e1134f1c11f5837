"""Parts a layer is put together from, chosen by the plan layer by layer."""

from .base import (Block, Embedding, FeedForward, Head, KVNeed, Mixer, Norm, Part, PositionEncoding, StateNeed, Stream,
                   TensorSpec, block_class, embedding_class, feed_forward_class, head_class, mixer_class, norm_class,
                   position_class, register_block, register_embedding, register_feed_forward, register_head,
                   register_mixer, register_norm, register_position)
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from .norm import Normed, RMSNorm
from .rope import RotaryTable
from .attention import GQAttention
from .mlp import SwiGLU
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding

__all__ = [n for n in dir() if not n.startswith("_")]
