from . import (attention, block, dense_feed_forward, embedding, feed_forward, head, layer_norm, min_gru, norm,  # noqa: F401
               parallel_block, rope, side_by_side, talking_attention)  # registers the built-in parts
from .base import MODES, Mixer, Part, Prenormed, RunContext, Runtime, as_delta
from .linear import add_linear, linear
from .registry import build_part, known_parts, register_part, unregister_part
