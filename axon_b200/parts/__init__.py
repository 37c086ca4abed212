"""Parts a model is put together from: mixers, feed-forwards, norms, position
encodings, blocks, embedding and head, each chosen per layer by the model's spec."""

from .base import (CATEGORIES, FeedForward, Mixer, Part, Runtime, StepContext, fold_owed, norm_owed,
                   part_class, register_part)
from .spec import (KvNeed, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, StateNeed, TensorDecl)
from . import standard  # registers the standard parts

__all__ = [
    "CATEGORIES", "FeedForward", "KvNeed", "LayerSpec", "Mixer", "ModelSpec", "Part", "PartSpec",
    "Runtime", "ScheduleEntry", "StateNeed", "StepContext", "TensorDecl", "fold_owed", "norm_owed",
    "part_class", "register_part",
]
