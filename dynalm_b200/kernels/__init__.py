"""Hand-written CUDA kernels (sources in ../csrc) and their Python faces."""
from . import lib, ops
from .gemm import linear

__all__ = ["lib", "ops", "linear"]
