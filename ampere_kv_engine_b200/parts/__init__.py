"""The parts a model is put together from.  Importing the package registers the built-in kinds."""

from . import (attention, block, embedding, feed_forward, gated_delta, norm, position,  # noqa: F401
               routed_experts)
