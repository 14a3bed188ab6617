"""Parts a model is put together from.  Importing the package registers the built-in
kinds; further kinds are added with `register_part` (see `base`)."""
from . import base
from .base import (Block, BuildContext, CacheNeed, FeedForward, KVNeed, LayerSpec, Mixer, ModelSpec, Norm, Part,
                   PartSpec, PositionEncoding, ScheduleEntry, StateNeed, WeightSpec, WeightStore, build_part,
                   known_parts, register_part)
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)
from .linear import Linear
