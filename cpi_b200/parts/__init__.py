from .base import (Part, Norm, Position, RotaryEncoding, ScoreBias, Mixer, FeedForward, Block, Junction, CacheView, build_part, registered,
                   register_norm, register_position, register_mixer, register_feed_forward, register_block, register_junction)
from .workspace import Workspace
from . import norms, positions, attention, latent, recurrent, parallel, feedforward, block, junction  # noqa: F401  (register the built-in kinds)
