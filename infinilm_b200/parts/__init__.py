from .base import (Arrangement, FeedForward, Mixer, Norm, Part, PositionEncoding, build_part, part_class,
                   register_part, unregister_part)
from .spec import CacheNeed, LayerSpec, ModelSpec, PartSpec, RunStep, WeightSpec
