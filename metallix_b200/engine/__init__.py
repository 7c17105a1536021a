"""Model, step function, scheduler, generation and trace replay."""
from .engine import Engine, StepEntry, StepError
from .model import DecoderModel

__all__ = ["Engine", "StepEntry", "StepError", "DecoderModel"]
