"""Parts a decoder is assembled from.  Importing this package registers the built-in kinds."""
from . import attention, block, mlp, norm, rope  # noqa: F401
from .base import (Block, CacheView, FeedForward, HostBatch, Mixer, Norm, Part, PositionEncoding, StepContext,
                   WeightSpec)
