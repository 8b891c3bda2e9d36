"""Parts of a model and their registries.  Importing this package registers the built-in kinds."""
from .base import (Block, CacheGroupView, FeedForward, KVCacheSpec, LayerCache, LayerCall, LayerSpec, Mixer, ModelSpec,
                   Norm, Part, PartSpec, PositionEncoding, StateSpec, StepContext, WeightSpec, build_part, part_class,
                   register_part)
from . import attention, block, embedding, linear, mlp, norm, rope  # noqa: F401  (registration)
