from .build import BuiltModel, build
from .context import CacheView, StepContext
from .model import Decoder
from .runtime import Runtime, parse_dtype
from .step import BatchBuilder, StepEntry, StepFunction
from .scheduler import Event, Request, Scheduler, SchedulerConfig
from .executor import GpuExecutor
from .engine import Engine, Generation, RequestStream

__all__ = ["BuiltModel", "build", "CacheView", "StepContext", "Decoder", "Runtime", "parse_dtype", "StepEntry",
           "StepFunction", "BatchBuilder", "Event", "Request", "Scheduler", "SchedulerConfig", "GpuExecutor", "Engine", "Generation", "RequestStream"]
