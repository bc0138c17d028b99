"""Error types of the engine.

The reference reports failures as `Status` codes (NotFound, Corrupt, Unsupported,
InvalidArgument, ResourceExhausted; dynacore/include/dynacore/base/status.h:19-32).
Here each code is an exception class so that callers can tell them apart.
"""


class EngineError(Exception):
    """Base class of every error the engine raises on purpose."""


class NotFound(EngineError):
    """A file, a config key or a tensor that should be there is not."""


class Corrupt(EngineError):
    """A file is there but its contents cannot be right."""


class Unsupported(EngineError):
    """Valid input that this engine refuses (another architecture, a size a kernel cannot take)."""


class InvalidArgument(EngineError):
    """A caller passed something out of range."""


class ResourceExhausted(EngineError):
    """The cache has no free page (or no free state slot) left."""


class ExtensionMissing(EngineError):
    """The CUDA extension could not be built or loaded; there is no other path."""
