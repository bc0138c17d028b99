"""dynalm_b200: a single-GPU inference engine for the dense Llama decoder, written for B200 (sm_100a)."""

from . import errors
from .errors import (Corrupt, EngineError, ExtensionMissing, InvalidArgument, NotFound, ResourceExhausted,
                     Unsupported)
from . import models as _models  # noqa: F401  registers architectures
from . import parts as _parts    # noqa: F401  registers part kinds
from .registry import find_architecture, register_architecture, registered_architectures

from .engine import Engine, Generation, Request, RequestStream, Scheduler, SchedulerConfig, StepEntry
from .sampling import SamplingParams

__version__ = "0.1.0"

__all__ = ["errors", "Corrupt", "EngineError", "ExtensionMissing", "InvalidArgument", "NotFound",
           "ResourceExhausted", "Unsupported", "find_architecture", "register_architecture",
           "registered_architectures", "Engine", "Generation", "Request", "RequestStream", "Scheduler",
           "SchedulerConfig", "StepEntry", "SamplingParams", "__version__"]
