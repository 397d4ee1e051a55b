"""Parts a decoder is assembled from.  Importing this package registers the
built-in parts."""

from . import registry  # noqa: F401
from . import norm, position, attention, feed_forward, block, embedding  # noqa: F401
from .registry import (register_block, register_embedding, register_feed_forward,  # noqa: F401
                       register_head, register_mixer, register_norm, register_position)
