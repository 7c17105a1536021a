"""Parts a decoder is put together from: mixers, feed-forwards, norms,
position encodings, block arrangements and the model's two ends."""
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register)
from .linear import Linear
from .registry import (CacheView, Prepared, Runtime, StepContext, StepPlan, WeightStore, build_part,
                       register_part, unregister_part)

__all__ = ["Linear", "CacheView", "Prepared", "Runtime", "StepContext", "StepPlan", "WeightStore",
           "build_part", "register_part", "unregister_part"]
