from .build import BuiltModel, build
from .context import CacheView, StepContext
from .model import Decoder
from .runtime import Runtime, parse_dtype
from .step import StepEntry, StepFunction

__all__ = ["BuiltModel", "build", "CacheView", "StepContext", "Decoder", "Runtime", "parse_dtype", "StepEntry",
           "StepFunction"]
