"""Parts that layers are put together from. Importing the package registers them."""
from . import attention, block, feed_forward, norm, position  # noqa: F401
from .base import CacheNeed, LayerCache, Part, StateNeed, StepContext  # noqa: F401
