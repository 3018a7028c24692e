from . import spec
from .base import (FeedForward, Mixer, Norm, Part, PositionEncoding, StepContext, to_device)
from .registry import (build_block, build_part, register_block, register_feed_forward, register_mixer,
                       register_norm, register_position)
from .linear import Linear, linear_forward
from . import norm, position, attention, feedforward, block, embedding   # register the built-in kinds
from .embedding import Embedding, Head
