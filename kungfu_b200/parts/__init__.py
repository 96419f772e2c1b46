"""Parts a model is composed of: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (Block, FeedForward, FixedState, Mixer, Norm, PagedKV, Part, PositionEncoding, StateNeed,
                   known, make, register_block, register_feed_forward, register_mixer, register_norm,
                   register_position)
from .norm import RmsNorm
from .rope import Rope
from .attention import PagedAttention
from .ffn import GatedFfn
from .embedding import Embedding, LmHead
from .block import SandwichBlock
from .model import DecoderModel, LayerCall, default_schedule
