"""Parts a model is assembled from: norms, position encodings, mixers, feed-forwards."""
from . import attention, moe, norm, position  # noqa: F401  (register the built-in kinds)
from .base import *  # noqa: F401,F403
