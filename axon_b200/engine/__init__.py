"""The model runner: a model built from its spec, the step function, the scheduler's driver."""

from .model import DecoderModel
from .step import Engine, OutOfPages, StepEntry, StepError

__all__ = ["DecoderModel", "Engine", "OutOfPages", "StepEntry", "StepError"]
