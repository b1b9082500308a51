"""Layer parts.  Importing this package registers the parts the LFM3 decoder is made of."""
from . import attention, block, ffn, norm, rope, shortconv  # noqa: F401  (registration)
from .base import (Block, FeedForward, Mixer, Norm, Part, Position, build_part, part_kinds,  # noqa: F401
                   register_part)
