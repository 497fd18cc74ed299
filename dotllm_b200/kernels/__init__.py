"""CUDA kernels for sm_100a and their Python wrappers (``ops``)."""
from . import ops  # noqa: F401
