"""Model layer: networks, the registry, the preprocessor and the single- / multi-step wrappers."""

from .preprocessor import Preprocessor2D
from .stepper import MultiStepWrapper, SingleStepWrapper
from . import model_registry  # noqa: F401

__all__ = ["Preprocessor2D", "SingleStepWrapper", "MultiStepWrapper", "model_registry"]
